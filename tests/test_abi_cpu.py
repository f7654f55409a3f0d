"""CPU tests of the boundary: the shared library loads without a GPU, exports
every symbol include/ullm_cuda.h declares, and fails loudly (no fallback)."""
import ctypes
import os
import re

import numpy as np
import pytest

from ullm_b200 import backend, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ullm_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ullm_cuda_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = backend.load_library()
    names = declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ullm_cuda.h but not exported"
    assert set(names) == set(backend.SIGNATURES), "python signature table out of sync with the header"


def test_gguf_header_and_library_agree():
    from ullm_b200 import gguf

    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "ullm_gguf.h")).read(), flags=re.S)
    names = sorted(set(re.findall(r"\b(ullm_gguf_[a-z0-9_]+)\s*\(", text)))
    lib = backend.load_library()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ullm_gguf.h but not exported"
    assert set(names) == set(gguf.SIGNATURES)


def test_safetensors_header_and_library_agree():
    from ullm_b200 import safetensors

    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "ullm_safetensors.h")).read(), flags=re.S)
    names = sorted(set(re.findall(r"\b(ullm_st_[a-z0-9_]+)\s*\(", text)))
    lib = backend.load_library()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ullm_safetensors.h but not exported"
    assert set(names) == set(safetensors.SIGNATURES)


def test_context_creation_without_device_is_unsupported():
    import torch  # only to learn whether this machine has a GPU

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(backend.Unsupported):
        backend.CudaContext(0)


def test_null_arguments_are_rejected_without_touching_cuda():
    lib = backend.load_library()
    assert lib.ullm_cuda_ctx_create(0, None) == backend.ERR_INVALID
    assert lib.ullm_cuda_matvec_quant(None, backend.Q4_K, None, 0, None, None, 0, 0) == backend.ERR_INVALID
    assert lib.ullm_cuda_synchronize(None) == backend.ERR_INVALID
    assert lib.ullm_cuda_buf_ptr(None) is None
    assert lib.ullm_cuda_last_error(None) == b"null context"


def test_generators_are_deterministic_and_in_range():
    a, b = synth.gen_q4k(8, 512, 42), synth.gen_q4k(8, 512, 42)
    assert np.array_equal(a, b) and a.shape == (8, 2 * 144)
    blk = a.reshape(-1, 144)
    d = blk[:, 0:4].copy().view(np.float16).astype(np.float32)
    assert d.min() >= 0.00099 and d.max() <= 0.0501
    w6 = synth.gen_q6k(8, 512, 42).reshape(-1, 210)
    d6 = w6[:, 208:210].copy().view(np.float16).astype(np.float32)
    assert d6.min() >= 0.00049 and d6.max() <= 0.01001
    x = synth.normal(7, 100000)
    assert abs(x.mean()) < 0.02 and abs(x.std() - 1) < 0.02
    assert np.array_equal(synth.splitmix64(5, 10, offset=90), synth.splitmix64(5, 100)[90:])
    r = synth.f32_to_bf16(np.array([1.0, 1.00390625, 3.14159], np.float32))
    assert synth.bf16_to_f32(r)[0] == 1.0 and abs(synth.bf16_to_f32(r)[2] - 3.14159) < 0.01
