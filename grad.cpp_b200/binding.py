"""ctypes mirror of include/gradb.h with the reference's class names.

``InferenceSession`` and ``TextGen`` follow the reference's C++ classes
(include/grad/transformer/inference.h:16-57, text_gen.h:12-38): same method
names, argument meaning and error behaviour (context overflow raises
RuntimeError, an id outside the vocabulary raises IndexError - the Python
spellings of std::runtime_error / std::out_of_range). Every call goes through
the C ABI; nothing here computes.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libgradb.so"

OK, ERR_CONTEXT_FULL, ERR_BAD_TOKEN, ERR_CHECKPOINT, ERR_CUDA, ERR_DEVICE_WAIT, ERR_INVALID, ERR_NO_DEVICE, \
    ERR_IO = range(9)
FP32, BF16 = 0, 1

_i32p = C.POINTER(C.c_int32)
_f32p = C.POINTER(C.c_float)


class ModelDesc(C.Structure):
    _fields_ = [("vocab_size", C.c_int32), ("d_model", C.c_int32), ("num_layers", C.c_int32),
                ("num_heads", C.c_int32), ("max_len", C.c_int32), ("arch", C.c_int32), ("d_ff", C.c_int32),
                ("dropout_rate", C.c_float), ("format_version", C.c_int32), ("has_fingerprint", C.c_int32),
                ("fingerprint_kind", C.c_uint32), ("fingerprint_hash", C.c_uint64)]


class Sampling(C.Structure):
    _fields_ = [("greedy", C.c_int32), ("temperature", C.c_float), ("repetition_penalty", C.c_float),
                ("top_k", C.c_int32), ("top_p", C.c_float)]


class GradbError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(message)
        self.status = status


# Every symbol include/gradb.h declares: name -> (restype, argtypes)
SIGNATURES = {
    "gradb_last_error": (C.c_char_p, []),
    "gradb_version": (C.c_char_p, []),
    "gradb_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "gradb_checkpoint_inspect": (C.c_int, [C.c_char_p, C.POINTER(ModelDesc)]),
    "gradb_tensor_count": (C.c_int, [C.POINTER(ModelDesc), C.POINTER(C.c_int)]),
    "gradb_tensor_shape": (C.c_int, [C.POINTER(ModelDesc), C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "gradb_checkpoint_write": (C.c_int, [C.c_char_p, C.POINTER(ModelDesc), C.POINTER(_f32p), C.c_int]),
    "gradb_model_load": (C.c_int, [C.c_char_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "gradb_model_from_host": (C.c_int, [C.POINTER(ModelDesc), C.POINTER(_f32p), C.c_int, C.c_int, C.c_int,
                                        C.POINTER(C.c_void_p)]),
    "gradb_model_save": (C.c_int, [C.c_void_p, C.c_char_p]),
    "gradb_model_describe": (C.c_int, [C.c_void_p, C.POINTER(ModelDesc)]),
    "gradb_model_free": (None, [C.c_void_p]),
    "gradb_session_create": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_void_p)]),
    "gradb_session_free": (None, [C.c_void_p]),
    "gradb_session_reset": (C.c_int, [C.c_void_p]),
    "gradb_session_position": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_int)]),
    "gradb_session_capacity": (C.c_int, [C.c_void_p]),
    "gradb_session_vocab": (C.c_int, [C.c_void_p]),
    "gradb_session_max_batch": (C.c_int, [C.c_void_p]),
    "gradb_step": (C.c_int, [C.c_void_p, _i32p, C.c_int, _f32p]),
    "gradb_prefill": (C.c_int, [C.c_void_p, _i32p, _i32p, C.c_int, _f32p]),
    "gradb_select": (C.c_int, [C.c_void_p, C.POINTER(Sampling), _f32p, C.c_int, _i32p]),
    "gradb_session_set_history": (C.c_int, [C.c_void_p, C.c_int, _i32p, C.c_int]),
    "gradb_select_from_logits": (C.c_int, [C.c_void_p, C.POINTER(Sampling), _f32p, _f32p, C.c_int, _i32p, _f32p]),
    "gradb_generate": (C.c_int, [C.c_void_p, _i32p, _i32p, C.c_int, C.POINTER(Sampling), C.c_int, _f32p, _i32p,
                                 C.c_int, _i32p, _f32p, _f32p]),
    "gradb_generate_stream": (C.c_int, [C.c_void_p, _i32p, _i32p, C.c_int, C.POINTER(Sampling), C.c_int, C.c_void_p,
                                        C.c_void_p, C.c_void_p, _i32p]),
    "gradb_session_admit": (C.c_int, [C.c_void_p, C.c_int, _i32p, _i32p, _i32p, _i32p, C.POINTER(_f32p), C.c_int,
                                      _i32p]),
    "gradb_session_decode": (C.c_int, [C.c_void_p, C.POINTER(Sampling), C.c_int, _i32p, C.c_int, _i32p, C.c_int, _i32p,
                                       _i32p]),
    "gradb_session_release": (C.c_int, [C.c_void_p, C.c_int]),
    "gradb_session_slot_ids": (C.c_int, [C.c_void_p, C.c_int, _i32p, C.c_int, C.POINTER(C.c_int)]),
    "gradb_score": (C.c_int, [C.c_void_p, _i32p, _i32p, C.c_int, C.c_int, _f32p, _f32p]),
    "gradb_mean_loss": (C.c_int, [C.c_void_p, _i32p, _i32p, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_double), _f32p,
                                  _f32p]),
    "gradb_session_last_ms": (C.c_int, [C.c_void_p, _f32p]),
    "gradb_session_cache_row": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, _f32p]),
    "gradb_attention_decode": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                       C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "gradb_attention_decode_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                              C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "gradb_attention_static_capacity": (C.c_int, []),
    "gradb_session_set_profiling": (C.c_int, [C.c_void_p, C.c_int]),
    "gradb_kernel_class_count": (C.c_int, []),
    "gradb_kernel_class_name": (C.c_char_p, [C.c_int]),
    "gradb_session_profile": (C.c_int, [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_uint64)]),
    "gradb_kernel_launches": (C.c_uint64, []),
}

# Only in the diagnostics build (libgradb_diag.so, csrc/gradb_diag.h); selected by GRADB_LIB=<path to that file>.
DIAG_SIGNATURES = {
    "gradb_session_stage_trace": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64), C.c_int, C.POINTER(C.c_int)]),
    "gradb_diag_attention_wait": (C.c_int, [C.c_void_p, C.c_uint, C.c_int]),
    "gradb_diag_count_nonfinite": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_longlong)]),
    "gradb_diag_poke_history": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int32]),
    "gradb_diag_wide_clocks": (C.c_int, [C.POINTER(C.c_uint64), C.c_int]),
    "gradb_diag_attn_clocks": (C.c_int, [C.POINTER(C.c_uint64), C.c_int]),
    "gradb_diag_select_clocks": (C.c_int, [C.POINTER(C.c_uint64), C.c_int]),
}

DRAW_FN = C.CFUNCTYPE(C.c_float, C.c_void_p, C.c_int)
TOKEN_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int32)

_lib = None


def lib():
    """Loads the CUDA library. There is no fallback: a missing build is an error."""
    global _lib
    if _lib is None:
        path = Path(os.environ.get("GRADB_LIB", LIB_PATH))
        if not path.exists():
            raise ImportError(f"{path} has not been built (python grad.cpp_b200/build.py); "
                              "this package has no CPU implementation")
        L = C.CDLL(str(path))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        for name, (res, args) in DIAG_SIGNATURES.items():
            if hasattr(L, name):
                fn = getattr(L, name)
                fn.restype = res
                fn.argtypes = args
        _lib = L
    return _lib


def _check(status):
    if status == OK:
        return
    msg = lib().gradb_last_error().decode()
    if status == ERR_BAD_TOKEN:
        raise IndexError(msg)            # std::out_of_range
    if status == ERR_CONTEXT_FULL:
        raise RuntimeError(msg)          # std::runtime_error
    raise GradbError(status, msg)


def _p(a, ty):
    return None if a is None else a.ctypes.data_as(ty)


def attention_decode(q, kcache, vcache, pos, max_len, splits, out, stream=0, fn="gradb_attention_decode"):
    """Stand-alone cached attention on torch CUDA tensors (device pointers are passed through).
    q/out: [n_seq, heads*64] float32; caches: [n_seq, heads, max_len, 64] float32; pos: [n_seq] int32."""
    n_seq, heads = kcache.shape[0], kcache.shape[1]
    _check(getattr(lib(), fn)(q.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), pos.data_ptr(), n_seq, heads, 64,
                              max_len, splits, out.data_ptr(), stream))
    return out


def inspect_checkpoint(path) -> ModelDesc:
    d = ModelDesc()
    _check(lib().gradb_checkpoint_inspect(str(path).encode(), C.byref(d)))
    return d


def write_checkpoint(path, desc: ModelDesc, tensors):
    arrs = [np.ascontiguousarray(t, np.float32) for t in tensors]
    ptrs = (_f32p * len(arrs))(*[_p(a, _f32p) for a in arrs])
    _check(lib().gradb_checkpoint_write(str(path).encode(), C.byref(desc), ptrs, len(arrs)))


class GPTModel:
    """Device-resident weights of one checkpoint (GPTModel::load / save)."""

    def __init__(self, handle):
        self._h = handle
        d = ModelDesc()
        _check(lib().gradb_model_describe(self._h, C.byref(d)))
        self.desc = d

    @classmethod
    def load(cls, path, device=0, precision=FP32):
        h = C.c_void_p()
        _check(lib().gradb_model_load(str(path).encode(), device, precision, C.byref(h)))
        return cls(h)

    @classmethod
    def from_host(cls, desc: ModelDesc, tensors, device=0, precision=FP32):
        arrs = [np.ascontiguousarray(t, np.float32) for t in tensors]
        ptrs = (_f32p * len(arrs))(*[_p(a, _f32p) for a in arrs])
        h = C.c_void_p()
        _check(lib().gradb_model_from_host(C.byref(desc), ptrs, len(arrs), device, precision, C.byref(h)))
        return cls(h)

    def save(self, path) -> bool:
        return lib().gradb_model_save(self._h, str(path).encode()) == OK

    def getVocabSize(self):
        return self.desc.vocab_size

    def getMaxLen(self):
        return self.desc.max_len

    def close(self):
        if self._h:
            lib().gradb_model_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown: the module's globals may already be gone
            pass


class BatchSession:
    """max_batch independent decode contexts on one stream."""

    def __init__(self, model: GPTModel, max_batch=1, max_len=0, stream=None):
        self.model = model
        h = C.c_void_p()
        _check(lib().gradb_session_create(model._h, max_batch, max_len, C.c_void_p(stream or 0), C.byref(h)))
        self._h = h
        self.max_batch = max_batch
        self.vocab = lib().gradb_session_vocab(h)

    def close(self):
        if self._h:
            lib().gradb_session_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown: the module's globals may already be gone
            pass

    def reset(self):
        _check(lib().gradb_session_reset(self._h))

    def position(self, seq=0):
        v = C.c_int()
        _check(lib().gradb_session_position(self._h, seq, C.byref(v)))
        return v.value

    def capacity(self):
        return lib().gradb_session_capacity(self._h)

    def step(self, tokens, want_logits=True):
        tk = np.ascontiguousarray(tokens, np.int32)
        out = np.empty((len(tk), self.vocab), np.float32) if want_logits else None
        _check(lib().gradb_step(self._h, _p(tk, _i32p), len(tk), _p(out, _f32p)))
        return out

    def prefill(self, prompts, want_logits=True):
        flat, offs = _flatten(prompts)
        out = np.empty((len(prompts), self.vocab), np.float32) if want_logits else None
        _check(lib().gradb_prefill(self._h, _p(flat, _i32p), _p(offs, _i32p), len(prompts), _p(out, _f32p)))
        return out

    def score(self, inputs, targets):
        """Teacher-forced scoring: (n_windows, seq_len) log-probabilities of the targets
        (0 where a target is outside the vocabulary). Device time in ``last_score_ms``."""
        inp = np.ascontiguousarray(inputs, np.int32)
        tgt = np.ascontiguousarray(targets, np.int32)
        if inp.ndim != 2 or tgt.shape != inp.shape:
            raise ValueError("inputs and targets must be (n_windows, seq_len) arrays of the same shape")
        out = np.empty(inp.shape, np.float32)
        ms = C.c_float(0)
        _check(lib().gradb_score(self._h, _p(inp, _i32p), _p(tgt, _i32p), inp.shape[0], inp.shape[1],
                                 _p(out, _f32p), C.cast(C.byref(ms), _f32p)))
        self.last_score_ms = float(ms.value)
        return out

    def mean_loss(self, inputs, targets, batch_windows=8):
        """training::mean_loss over in-memory windows: (mean loss, per-batch losses)."""
        inp = np.ascontiguousarray(inputs, np.int32)
        tgt = np.ascontiguousarray(targets, np.int32)
        if inp.ndim != 2 or tgt.shape != inp.shape:
            raise ValueError("inputs and targets must be (n_windows, seq_len) arrays of the same shape")
        n, S = inp.shape
        nb = (n + batch_windows - 1) // max(batch_windows, 1)
        batch = np.zeros(max(nb, 1), np.float32)
        mean = C.c_double(0)
        ms = C.c_float(0)
        _check(lib().gradb_mean_loss(self._h, _p(inp, _i32p), _p(tgt, _i32p), n, S, batch_windows, C.byref(mean),
                                     _p(batch, _f32p), C.cast(C.byref(ms), _f32p)))
        self.last_score_ms = float(ms.value)
        return float(mean.value), batch[:nb].copy()

    def select(self, sampling: Sampling, uniforms=None, n_seq=None, logits=None, want_probs=False):
        n = n_seq if n_seq is not None else (len(logits) if logits is not None else self.max_batch)
        u = None if uniforms is None else np.ascontiguousarray(uniforms, np.float32)
        out = np.empty(n, np.int32)
        if logits is None:
            _check(lib().gradb_select(self._h, C.byref(sampling), _p(u, _f32p), n, _p(out, _i32p)))
            return out
        lg = np.ascontiguousarray(logits, np.float32)
        probs = np.empty((n, self.vocab), np.float32) if want_probs else None
        _check(lib().gradb_select_from_logits(self._h, C.byref(sampling), _p(lg, _f32p), _p(u, _f32p), n,
                                              _p(out, _i32p), _p(probs, _f32p)))
        return (out, probs) if want_probs else out

    def set_history(self, seq, ids):
        a = np.ascontiguousarray(ids, np.int32)
        _check(lib().gradb_session_set_history(self._h, seq, _p(a, _i32p), len(a)))

    def generate(self, prompts, sampling: Sampling, max_new, uniforms=None, timings=False):
        flat, offs = _flatten(prompts)
        n = len(prompts)
        stride = max((len(p) for p in prompts), default=0) + max_new + 1
        out = np.zeros((n, stride), np.int32)
        lens = np.zeros(n, np.int32)
        u = None if uniforms is None else np.ascontiguousarray(uniforms, np.float32).reshape(n, max_new)
        step_ms = np.zeros(max(max_new, 1), np.float32)
        pre_ms = C.c_float(0)
        _check(lib().gradb_generate(self._h, _p(flat, _i32p), _p(offs, _i32p), n, C.byref(sampling), max_new,
                                    _p(u, _f32p), _p(out, _i32p), stride, _p(lens, _i32p), _p(step_ms, _f32p),
                                    C.byref(pre_ms)))
        seqs = [out[i, :lens[i]].copy() for i in range(n)]
        if timings:
            return seqs, step_ms, float(pre_ms.value)
        return seqs

    def generate_stream(self, prompts, sampling: Sampling, max_new, on_token, draw=None):
        """gradb_generate_stream: on_token(seq, index, id) is called as each id is chosen (a true return value ends
        that sequence); draw(seq) supplies one uniform per sampled id, asked for right before it is needed.
        Returns the ids handed out per sequence."""
        flat, offs = _flatten(prompts)
        n = len(prompts)
        emitted = np.zeros(n, np.int32)
        failure = []

        def _tok(_user, seq, index, token):
            try:
                return 1 if on_token(seq, index, token) else 0
            except BaseException as e:  # must not unwind through the C frames
                failure.append(e)
                return 1

        def _draw(_user, seq):
            try:
                return float(draw(seq))
            except BaseException as e:
                failure.append(e)
                return 0.0

        tok_cb = TOKEN_FN(_tok)
        draw_cb = DRAW_FN(_draw) if draw is not None else None
        _check(lib().gradb_generate_stream(self._h, _p(flat, _i32p), _p(offs, _i32p), n, C.byref(sampling), max_new,
                                           C.cast(draw_cb, C.c_void_p) if draw_cb else None,
                                           C.cast(tok_cb, C.c_void_p), None, _p(emitted, _i32p)))
        if failure:
            raise failure[0]
        return emitted

    def admit(self, slots, prompts, max_new, uniforms=None, reuse_prefix=False):
        """gradb_session_admit: starts prompts[i] in slot slots[i]; returns the cached positions kept per prompt."""
        flat, offs = _flatten(prompts)
        n = len(prompts)
        sl = np.ascontiguousarray(slots, np.int32)
        mn = np.ascontiguousarray(np.broadcast_to(max_new, (n,)), np.int32)
        reused = np.zeros(n, np.int32)
        uptr = None
        if uniforms is not None:
            keep = [None if u is None else np.ascontiguousarray(u, np.float32) for u in uniforms]
            uptr = (_f32p * n)(*[_p(u, _f32p) if u is not None else None for u in keep])
        _check(lib().gradb_session_admit(self._h, n, _p(sl, _i32p), _p(flat, _i32p), _p(offs, _i32p), _p(mn, _i32p), uptr,
                                         int(reuse_prefix), _p(reused, _i32p)))
        return reused

    def decode(self, sampling: Sampling, n_steps, stop_ids=()):
        """gradb_session_decode: ([new ids per slot], finished flags) for n_steps iterations over the live slots."""
        B = self.max_batch
        out = np.zeros((B, n_steps), np.int32)
        cnt = np.zeros(B, np.int32)
        fin = np.zeros(B, np.int32)
        st = np.ascontiguousarray(stop_ids, np.int32) if len(stop_ids) else None
        _check(lib().gradb_session_decode(self._h, C.byref(sampling), n_steps, _p(st, _i32p), len(stop_ids),
                                          _p(out, _i32p), n_steps, _p(cnt, _i32p), _p(fin, _i32p)))
        return [out[b, :cnt[b]].copy() for b in range(B)], fin.astype(bool)

    def release(self, slot):
        _check(lib().gradb_session_release(self._h, slot))

    def slot_ids(self, slot):
        n = C.c_int()
        buf = np.zeros(self.capacity() + 2, np.int32)
        _check(lib().gradb_session_slot_ids(self._h, slot, _p(buf, _i32p), len(buf), C.byref(n)))
        return buf[:n.value].copy()

    def set_profiling(self, on: bool):
        _check(lib().gradb_session_set_profiling(self._h, int(on)))

    def profile(self):
        """{kernel class: (total ms, launches)} accumulated since profiling was switched on."""
        n = lib().gradb_kernel_class_count()
        ms = (C.c_double * n)()
        cnt = (C.c_uint64 * n)()
        _check(lib().gradb_session_profile(self._h, ms, cnt))
        return {lib().gradb_kernel_class_name(i).decode(): (ms[i], int(cnt[i])) for i in range(n)}

    def stage_trace(self):
        """Diagnostics build only."""
        buf = (C.c_uint64 * 1024)()
        n = C.c_int()
        _check(lib().gradb_session_stage_trace(self._h, buf, 1024, C.byref(n)))
        return np.array(buf[:n.value], np.uint64)

    def diag_attention_wait(self, spin_limit, skip_tile):
        """Diagnostics build only: make the attention kernel's tile wait expire (gradb_diag.h)."""
        _check(lib().gradb_diag_attention_wait(self._h, spin_limit, skip_tile))

    def diag_count_nonfinite(self, n_seq):
        n = C.c_longlong()
        _check(lib().gradb_diag_count_nonfinite(self._h, n_seq, C.byref(n)))
        return int(n.value)

    def diag_poke_history(self, seq, index, token):
        _check(lib().gradb_diag_poke_history(self._h, seq, index, token))

    def last_ms(self):
        v = C.c_float()
        _check(lib().gradb_session_last_ms(self._h, C.byref(v)))
        return float(v.value)

    def cache_row(self, seq, layer, which, pos):
        out = np.empty(self.model.desc.d_model, np.float32)
        _check(lib().gradb_session_cache_row(self._h, seq, layer, which, pos, _p(out, _f32p)))
        return out


def _flatten(prompts):
    offs = np.zeros(len(prompts) + 1, np.int32)
    for i, p in enumerate(prompts):
        offs[i + 1] = offs[i] + len(p)
    flat = np.zeros(max(int(offs[-1]), 1), np.int32)
    for i, p in enumerate(prompts):
        flat[offs[i]:offs[i + 1]] = np.asarray(p, np.int32)
    return flat, offs


class InferenceSession:
    """One sequence; mirrors grad::InferenceSession (inference.h:16-57)."""

    def __init__(self, model: GPTModel):
        self._s = BatchSession(model, 1)

    def step(self, token_id: int):
        """Appends token_id and returns the next-token logits (vocab floats)."""
        return self._s.step([int(token_id)])[0]

    def position(self):
        return self._s.position(0)

    def capacity(self):
        return self._s.capacity()

    def vocabSize(self):
        return self._s.vocab


class TextGen:
    """Mirrors grad::TextGen (text_gen.h:12-38) with ids in and ids out.

    The reference draws from a process-wide generator that cannot be seeded
    through its API; here the uniform draws are an explicit argument."""

    def __init__(self, model: GPTModel):
        self.model = model
        self._s = BatchSession(model, 1)

    def generate_greedy(self, prompt_tokens, max_tokens=50, repetition_penalty=1.2):
        if len(prompt_tokens) == 0:
            return np.zeros(0, np.int32)
        sp = Sampling(1, 1.0, repetition_penalty, 0, 1.0)
        return self._s.generate([prompt_tokens], sp, max_tokens)[0]

    def generate_sample(self, prompt_tokens, temperature=1.0, max_tokens=50, repetition_penalty=1.2, top_k=0,
                        top_p=1.0, draws=None, rng=None):
        if len(prompt_tokens) == 0:
            return np.zeros(0, np.int32)
        if draws is None:
            rng = rng or np.random.default_rng()
            draws = rng.random(max_tokens, dtype=np.float32)
        sp = Sampling(0, temperature, repetition_penalty, top_k, top_p)
        return self._s.generate([prompt_tokens], sp, max_tokens, uniforms=np.asarray(draws, np.float32)[:max_tokens]
                                if len(draws) >= max_tokens else np.pad(np.asarray(draws, np.float32),
                                                                        (0, max_tokens - len(draws))))[0]

    def generate_stream(self, prompt_tokens, on_token, temperature=1.0, max_tokens=50, repetition_penalty=1.2,
                        top_k=0, top_p=1.0, draws=None, rng=None):
        """on_token(id) runs as each id is chosen (text_gen.cpp:107-116); returns how many were generated."""
        if len(prompt_tokens) == 0:
            return 0
        it = iter(draws) if draws is not None else None
        rng = rng or np.random.default_rng()
        draw = (lambda seq: next(it)) if it is not None else (lambda seq: rng.random(dtype=np.float32))
        sp = Sampling(0, temperature, repetition_penalty, top_k, top_p)
        n = self._s.generate_stream([prompt_tokens], sp, max_tokens, lambda seq, i, t: on_token(int(t)), draw)
        return int(n[0])
