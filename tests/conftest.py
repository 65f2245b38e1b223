"""Shared fixtures. GPU tests are marked ``gpu``; everything else runs on CPU."""
from __future__ import annotations

import importlib.util
import sys
import zlib
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def load_package():
    """The package directory is named after the reference project and contains a
    dot, so it is loaded by path under the importable alias ``grad_cpp_b200``."""
    if "grad_cpp_b200" in sys.modules:
        return sys.modules["grad_cpp_b200"]
    pkg_dir = ROOT / "grad.cpp_b200"
    spec = importlib.util.spec_from_file_location("grad_cpp_b200", pkg_dir / "__init__.py",
                                                  submodule_search_locations=[str(pkg_dir)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["grad_cpp_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def ck(pkg):
    from grad_cpp_b200 import checkpoint
    return checkpoint


@pytest.fixture(scope="session")
def golden():
    return np.load(ROOT / "tests" / "golden" / "decode_golden.npz")


@pytest.fixture(scope="session")
def port():
    from oracle.oracle import Port
    return Port()


@pytest.fixture(scope="session")
def port64():
    from oracle.oracle import Port
    return Port(double=True)


# Mirrors tests/golden/make_golden.py: name -> (dims tuple, seed, std, perturb)
GOLDEN_MODELS = {
    "tiny_gpt2": ((23, 32, 2, 4, 16, 0), 101, 0.3, True),
    "tiny_modern": ((23, 32, 2, 4, 16, 1), 102, 0.3, True),
    "hs64_gpt2": ((301, 128, 2, 2, 40, 0), 103, 0.08, True),
    "hs64_modern": ((301, 128, 3, 2, 40, 1), 104, 0.08, True),
    "odd_modern": ((1003, 192, 2, 3, 24, 1), 105, 0.05, False),
}


@pytest.fixture(scope="session")
def golden_ckpt(ck, golden, tmp_path_factory):
    """Regenerates a golden model's checkpoint from its seed and checks the
    bytes against the CRC recorded when the fixture was made."""
    cache = {}
    base = tmp_path_factory.mktemp("ckpt")

    def get(name):
        if name not in cache:
            dims, seed, std, perturb = GOLDEN_MODELS[name]
            dm = ck.ModelDims(*dims)
            path = base / f"{name}.bin"
            ck.write_synthetic(path, dm, seed, std, perturb)
            assert zlib.crc32(path.read_bytes()) == int(golden[f"{name}/file_crc"][0]), \
                "seeded weights no longer reproduce the fixture's checkpoint"
            cache[name] = (dm, str(path))
        return cache[name]

    return get


def sampler_logits(seed, vocab, scale, quantum):
    rng = np.random.default_rng(int(seed))
    x = rng.standard_normal(int(vocab), dtype=np.float32) * np.float32(scale)
    if quantum > 0:
        x = (np.round(x / np.float32(quantum)) * np.float32(quantum)).astype(np.float32)
    return x
