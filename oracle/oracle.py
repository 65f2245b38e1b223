"""ctypes bindings for the two CPU checkers. TEST INFRASTRUCTURE ONLY.

* ``Port``  - this repository's plain-C restatement (oracle/decode_oracle.c),
  in float (``libgradoracle.so``) or with double intermediates
  (``libgradoracle64.so``).
* ``Ref``   - the reference's own decode path compiled unmodified
  (oracle/_ref/libgradref.so), when it has been built.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import
this module; the product library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int)


def _ptr(a, ty):
    return a.ctypes.data_as(ty) if a is not None else None


def build_port() -> None:
    subprocess.run(["make", "-C", str(HERE), "port"], check=True, capture_output=True)


def build_ref(reference_root: str | None = None) -> bool:
    """Builds oracle/_ref from the grad.cpp tree at `reference_root` (else the one GRADREF_ROOT names), when that
    tree is present. Returns whether the compiled reference is available afterwards."""
    reference_root = reference_root or os.environ.get("GRADREF_ROOT")
    if reference_root and Path(reference_root).is_dir():
        subprocess.run(["make", "-C", str(HERE), "-j8", "ref", f"REF={reference_root}"], check=True,
                       capture_output=True)
    return ref_available()


def ref_available() -> bool:
    return (HERE / "_ref" / "libgradref.so").exists()


def _mean_loss(fn, m, inputs, targets, batch_windows):
    inp = np.ascontiguousarray(inputs, np.int32)
    tgt = np.ascontiguousarray(targets, np.int32)
    n, S = inp.shape
    assert tgt.shape == inp.shape
    nb = (n + batch_windows - 1) // batch_windows
    mean = C.c_double(0)
    batch = np.zeros(max(nb, 1), np.float32)
    logp = np.zeros((n, S), np.float32)
    rc = fn(m, _ptr(inp, _i32p), _ptr(tgt, _i32p), n, S, batch_windows, C.byref(mean), _ptr(batch, _f32p),
            _ptr(logp, _f32p))
    if rc:
        raise RuntimeError(f"mean_loss failed rc={rc}")
    return float(mean.value), batch[:nb].copy(), logp


class Port:
    """The restated algorithm. ``double=True`` selects the double-precision witness."""

    def __init__(self, double: bool = False):
        name = "libgradoracle64.so" if double else "libgradoracle.so"
        path = HERE / name
        if not path.exists():
            build_port()
        self.pre = "gro64_" if double else "gro_"
        L = self.L = C.CDLL(str(path))
        f = self._f
        f("model_load").restype = C.c_void_p
        f("model_load").argtypes = [C.c_char_p, C.c_char_p, C.c_size_t]
        f("model_free").argtypes = [C.c_void_p]
        f("model_dims").argtypes = [C.c_void_p, _i32p]
        f("model_fingerprint_hash").restype = C.c_uint64
        f("model_fingerprint_hash").argtypes = [C.c_void_p]
        f("session_new").restype = C.c_void_p
        f("session_new").argtypes = [C.c_void_p]
        f("session_free").argtypes = [C.c_void_p]
        f("session_reset").argtypes = [C.c_void_p]
        f("session_position").argtypes = [C.c_void_p]
        f("session_step").argtypes = [C.c_void_p, C.c_int, _f32p]
        f("session_cache_row").argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, _f32p]
        f("generate").argtypes = [C.c_void_p, _i32p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float,
                                  C.c_int, C.c_float, _f32p, _i32p, C.c_int]
        f("mean_loss").argtypes = [C.c_void_p, _i32p, _i32p, C.c_int, C.c_int, C.c_int,
                                   C.POINTER(C.c_double), _f32p, _f32p]
        L.gro_apply_penalty.argtypes = [_f32p, C.c_int, _i32p, C.c_int, C.c_float]
        L.gro_argmax.argtypes = [_f32p, C.c_int]
        L.gro_sample.argtypes = [_f32p, C.c_int, C.c_float, C.c_int, C.c_float, C.c_float, _f32p]

    def _f(self, name):
        return getattr(self.L, self.pre + name)

    # -- model / session -------------------------------------------------
    def load(self, path: str):
        err = C.create_string_buffer(1024)
        m = self._f("model_load")(str(path).encode(), err, 1024)
        if not m:
            raise RuntimeError(err.value.decode())
        return m

    def free(self, m):
        self._f("model_free")(m)

    def dims(self, m):
        d = np.zeros(9, np.int32)
        self._f("model_dims")(m, _ptr(d, _i32p))
        keys = ["vocab", "d_model", "layers", "heads", "max_len", "arch", "d_ff", "has_fp", "fp_kind"]
        out = dict(zip(keys, (int(v) for v in d)))
        out["fp_hash"] = int(self._f("model_fingerprint_hash")(m))
        return out

    def session(self, m):
        return self._f("session_new")(m)

    def session_free(self, s):
        self._f("session_free")(s)

    def step(self, s, token: int, vocab: int):
        out = np.empty(vocab, np.float32)
        rc = self._f("session_step")(s, int(token), _ptr(out, _f32p))
        return rc, out

    def cache_row(self, s, layer, which, pos, d):
        out = np.empty(d, np.float32)
        self._f("session_cache_row")(s, layer, which, pos, _ptr(out, _f32p))
        return out

    def logits_for(self, m, tokens):
        """Teacher-forced: feeds tokens one by one, returns (len, vocab) logits."""
        V = self.dims(m)["vocab"]
        s = self.session(m)
        rows = []
        for t in tokens:
            rc, lg = self.step(s, t, V)
            assert rc == 0, rc
            rows.append(lg)
        self.session_free(s)
        return np.stack(rows)

    def generate(self, m, prompt, max_tokens, greedy=True, temperature=1.0, penalty=1.2, top_k=0,
                 top_p=1.0, draws=None):
        prompt = np.ascontiguousarray(prompt, np.int32)
        cap = len(prompt) + max_tokens + 1
        out = np.zeros(cap, np.int32)
        dr = None if draws is None else np.ascontiguousarray(draws, np.float32)
        n = self._f("generate")(m, _ptr(prompt, _i32p), len(prompt), max_tokens, int(greedy),
                                temperature, penalty, top_k, top_p, _ptr(dr, _f32p), _ptr(out, _i32p), cap)
        if n < 0:
            raise RuntimeError(f"oracle generate failed rc={-n}")
        return out[:n].copy()

    def mean_loss(self, m, inputs, targets, batch_windows=8):
        """Teacher-forced scoring: (mean loss, per-batch losses, per-row target log-probabilities)."""
        return _mean_loss(self._f("mean_loss"), m, inputs, targets, batch_windows)

    # -- selection stage ---------------------------------------------------
    def apply_penalty(self, logits, tokens, penalty):
        lg = np.array(logits, np.float32, copy=True)
        tk = np.ascontiguousarray(tokens, np.int32)
        self.L.gro_apply_penalty(_ptr(lg, _f32p), len(lg), _ptr(tk, _i32p), len(tk), penalty)
        return lg

    def argmax(self, logits):
        lg = np.ascontiguousarray(logits, np.float32)
        return int(self.L.gro_argmax(_ptr(lg, _f32p), len(lg)))

    def sample(self, logits, temperature, top_k, top_p, u, want_probs=False):
        lg = np.ascontiguousarray(logits, np.float32)
        probs = np.empty_like(lg) if want_probs else None
        tok = int(self.L.gro_sample(_ptr(lg, _f32p), len(lg), temperature, top_k, top_p, u,
                                    _ptr(probs, _f32p)))
        return (tok, probs) if want_probs else tok


class Ref:
    """The compiled reference. The sampler's generator is process-wide and is
    seeded from GRADREF_SEED the first time it is used, so set the seed (or the
    environment variable) before the first sampling call of the process."""

    def __init__(self, seed: int | None = None):
        if seed is not None:
            os.environ["GRADREF_SEED"] = str(int(seed))
        L = self.L = C.CDLL(str(HERE / "_ref" / "libgradref.so"))
        L.gradref_last_error.restype = C.c_char_p
        L.gradref_model_load.restype = C.c_void_p
        L.gradref_model_load.argtypes = [C.c_char_p]
        L.gradref_model_new.restype = C.c_void_p
        L.gradref_model_new.argtypes = [C.c_int] * 6
        L.gradref_model_save.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_uint, C.c_ulonglong]
        L.gradref_model_free.argtypes = [C.c_void_p]
        L.gradref_model_dims.argtypes = [C.c_void_p, _i32p]
        L.gradref_session_new.restype = C.c_void_p
        L.gradref_session_new.argtypes = [C.c_void_p]
        L.gradref_session_free.argtypes = [C.c_void_p]
        L.gradref_session_position.argtypes = [C.c_void_p]
        L.gradref_session_step.argtypes = [C.c_void_p, C.c_int, _f32p]
        L.gradref_generate_greedy.argtypes = [C.c_void_p, _i32p, C.c_int, C.c_int, C.c_float, _i32p, C.c_int]
        gs = [C.c_void_p, _i32p, C.c_int, C.c_float, C.c_int, C.c_float, C.c_int, C.c_float, _i32p,
              C.c_int, _f32p]
        L.gradref_generate_sample.argtypes = gs
        L.gradref_generate_stream.argtypes = gs
        L.gradref_sample_from_logits.argtypes = [C.c_void_p, _f32p, C.c_int, C.c_float, C.c_int,
                                                 C.c_float, _f32p]
        L.gradref_mean_loss.argtypes = [C.c_void_p, _i32p, _i32p, C.c_int, C.c_int, C.c_int,
                                        C.POINTER(C.c_double), _f32p, _f32p]
        L.gradref_tokenfile_write.argtypes = [C.c_char_p, _i32p, C.c_ulonglong, C.c_int]
        L.gradref_dataset_open.argtypes = [C.c_char_p, C.c_int, C.c_int, C.POINTER(C.c_ulonglong)]
        L.gradref_loader_windows.restype = C.c_longlong
        L.gradref_loader_windows.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint, C.c_int,
                                             _i32p, _i32p, C.c_longlong]

    def load(self, path):
        # The reference prints a success line to stdout from load(); keep it off ours.
        m = self.L.gradref_model_load(str(path).encode())
        if not m:
            raise RuntimeError(self.L.gradref_last_error().decode())
        return m

    def new(self, vocab, d_model, layers, heads, max_len, modern):
        return self.L.gradref_model_new(vocab, d_model, layers, heads, max_len, int(modern))

    def save(self, m, path, fingerprint=None):
        kind, h = fingerprint if fingerprint else (0, 0)
        return self.L.gradref_model_save(m, str(path).encode(), int(fingerprint is not None), kind, h)

    def free(self, m):
        self.L.gradref_model_free(m)

    def dims(self, m):
        d = np.zeros(7, np.int32)
        self.L.gradref_model_dims(m, _ptr(d, _i32p))
        keys = ["vocab", "d_model", "layers", "heads", "max_len", "arch", "d_ff"]
        return dict(zip(keys, (int(v) for v in d)))

    def session(self, m):
        return self.L.gradref_session_new(m)

    def session_free(self, s):
        self.L.gradref_session_free(s)

    def step(self, s, token, vocab, want=True):
        out = np.empty(vocab, np.float32) if want else None
        rc = self.L.gradref_session_step(s, int(token), _ptr(out, _f32p))
        return rc, out

    def logits_for(self, m, tokens):
        V = self.dims(m)["vocab"]
        s = self.session(m)
        rows = []
        for t in tokens:
            rc, lg = self.step(s, t, V)
            assert rc == 0, rc
            rows.append(lg)
        self.session_free(s)
        return np.stack(rows)

    def generate_greedy(self, m, prompt, max_tokens, penalty=1.2):
        prompt = np.ascontiguousarray(prompt, np.int32)
        cap = len(prompt) + max_tokens + 1
        out = np.zeros(cap, np.int32)
        n = self.L.gradref_generate_greedy(m, _ptr(prompt, _i32p), len(prompt), max_tokens, penalty,
                                           _ptr(out, _i32p), cap)
        return out[:n].copy()

    def generate_sample(self, m, prompt, temperature, max_tokens, penalty=1.2, top_k=0, top_p=1.0,
                        stream=False):
        prompt = np.ascontiguousarray(prompt, np.int32)
        cap = len(prompt) + max_tokens + 1
        out = np.zeros(cap, np.int32)
        draws = np.zeros(max_tokens + 1, np.float32)
        fn = self.L.gradref_generate_stream if stream else self.L.gradref_generate_sample
        n = fn(m, _ptr(prompt, _i32p), len(prompt), temperature, max_tokens, penalty, top_k, top_p,
               _ptr(out, _i32p), cap, _ptr(draws, _f32p))
        n_gen = n if stream else n - len(prompt)
        return out[:n].copy(), draws[:n_gen].copy()

    def mean_loss(self, m, inputs, targets, batch_windows=8):
        """The reference's full-sequence forward + cross_entropy, batched as `grad eval` does."""
        return _mean_loss(self.L.gradref_mean_loss, m, inputs, targets, batch_windows)

    # -- token files and batch assembly (src/data) -------------------------
    def tokenfile_write(self, path, ids, vocab):
        a = np.ascontiguousarray(ids, np.int32)
        if self.L.gradref_tokenfile_write(str(path).encode(), _ptr(a, _i32p), len(a), vocab):
            raise RuntimeError(self.L.gradref_last_error().decode())

    def dataset_open(self, path, seq_length, stride):
        """(windows, vocab, token count) as MappedTokenDataset reports them; raises with its message."""
        info = (C.c_ulonglong * 3)()
        if self.L.gradref_dataset_open(str(path).encode(), seq_length, stride, info):
            raise RuntimeError(self.L.gradref_last_error().decode())
        return int(info[0]), int(info[1]), int(info[2])

    def loader_windows(self, path, seq_length, stride, batch_size, shuffle, seed, max_batches, cap=1 << 16):
        inp = np.zeros((cap, seq_length), np.int32)
        tgt = np.zeros((cap, seq_length), np.int32)
        n = self.L.gradref_loader_windows(str(path).encode(), seq_length, stride, batch_size, int(shuffle), seed,
                                          max_batches, _ptr(inp, _i32p), _ptr(tgt, _i32p), cap)
        if n < 0:
            raise RuntimeError(self.L.gradref_last_error().decode())
        assert n <= cap
        return inp[:n].copy(), tgt[:n].copy()

    def sample_from_logits(self, m, logits, temperature, top_k, top_p):
        lg = np.ascontiguousarray(logits, np.float32)
        u = C.c_float(0)
        tok = self.L.gradref_sample_from_logits(m, _ptr(lg, _f32p), len(lg), temperature, top_k, top_p,
                                                C.byref(u))
        return int(tok), float(u.value)
