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


# ---- the Rust crate a maintainer adds beside crates/ullm-metal (source only: no Rust toolchain here) ----
CRATE = os.path.join(ROOT, "crates", "ullm-cuda")

# Public fields of the six input types ullm-model builds (crates/ullm-metal/src/forward.rs:24-110), in order.
REFERENCE_TYPES = {
    "GpuParams": ["n_embd", "n_layer", "n_head", "n_kv_head", "head_dim", "n_ff", "n_ctx", "vocab", "rope_theta", "eps", "rope_neox", "qk_norm",
                  "sandwich_norm", "geglu", "n_experts", "n_experts_used", "moe_inter", "sliding_window"],
    "GpuWeight": ["dtype", "bytes", "out", "cols", "mlx_scales", "mlx_biases", "mlx_group"],
    "GpuExperts": ["bytes", "scales", "biases", "n_experts", "out", "cols", "group"],
    "GpuLayerInput": ["attn_norm", "wq", "wk", "wv", "wo", "q_bias", "k_bias", "v_bias", "q_norm", "k_norm", "post_attn_norm", "post_ffn_norm",
                      "ffn_norm", "w_gate", "w_up", "w_down", "moe_gate", "experts_gate", "experts_up", "experts_down"],
    "GpuModelInput": ["params", "output", "final_norm", "layers"],
}


def test_rust_bindings_are_what_the_headers_say():
    """src/ffi.rs is generated from include/*.h; a header edit without regenerating it fails here."""
    import subprocess
    import sys

    r = subprocess.run([sys.executable, os.path.join(CRATE, "gen_ffi.py"), "--check"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    ffi = open(os.path.join(CRATE, "src", "ffi.rs")).read()
    fns = set(re.findall(r"pub fn (ullm_[a-z0-9_]+)\(", ffi))
    assert set(declared_symbols()) <= fns
    # struct members: same names in the same order as the C declarations
    hdr = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "ullm_cuda.h")).read(), flags=re.S)
    for name in ("ullm_gpu_params", "ullm_gpu_weight", "ullm_gpu_layer_input", "ullm_gpu_model_input", "ullm_moe_experts_input", "ullm_chain_op",
                 "ullm_shard_op", "ullm_debug_stat"):
        body = re.search(r"typedef\s+struct\s*\w*\s*\{([^{}]*)\}\s*" + name + r"\s*;", hdr).group(1)
        c_fields = []
        for stmt in body.split(";"):
            for part in stmt.split(","):
                mm = re.search(r"([A-Za-z_][A-Za-z0-9_]*)\s*(\[[^\]]*\])?\s*$", part.strip())
                if mm and part.strip():
                    c_fields.append(mm.group(1))
        rust = re.search(r"pub struct " + name + r" \{(.*?)\n\}", ffi, flags=re.S).group(1)
        r_fields = [f.replace("r#", "") for f in re.findall(r"pub ([a-z_0-9#]+):", rust)]
        assert r_fields == c_fields, name


def test_rust_crate_mirrors_the_reference_surface():
    """lib.rs exports the reference backend's names with the reference's fields, so that ullm-model's
    `use ullm_metal::{...}` (crates/ullm-model/src/lib.rs:20) becomes `use ullm_cuda::{...}` and nothing else."""
    lib_rs = open(os.path.join(CRATE, "src", "lib.rs")).read()
    for name, fields in REFERENCE_TYPES.items():
        body = re.search(r"pub struct " + name + r"(?:<'a>)? \{(.*?)\n\}", lib_rs, flags=re.S).group(1)
        assert re.findall(r"pub ([a-z_0-9]+):", body) == fields, name
    for method in ("pub fn new(input: &GpuModelInput) -> Result<Self>", "pub fn forward(&self, x_init: &[f32], pos: usize) -> Result<Vec<f32>>",
                   "pub fn forward_batch(&self, embeds: &[f32], s: usize) -> Result<Vec<f32>>", "pub fn supports_batched_prefill(&self) -> bool",
                   "pub fn forward_debug(&self, x_init: &[f32], pos: usize)", "pub fn device_name(&self) -> String", "pub fn upload(&self, bytes: &[u8]) -> Buffer",
                   "pub fn matvec_quant(", "pub fn matvec_resident(", "pub fn matvec_mlx4(", "pub fn matmul_mlx4("):
        assert method in lib_rs, method
    # every ffi function the wrapper calls exists in the generated bindings
    ffi = open(os.path.join(CRATE, "src", "ffi.rs")).read()
    for fn in set(re.findall(r"ffi::(ullm_[a-z0-9_]+)\(", lib_rs)):
        assert f"pub fn {fn}(" in ffi, fn
    for f in ("Cargo.toml", "build.rs"):
        assert os.path.exists(os.path.join(CRATE, f))
