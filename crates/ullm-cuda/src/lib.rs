//! CUDA (NVIDIA B200, sm_100a) compute backend for uLLM: the public surface of `ullm-metal`
//! (`crates/ullm-metal/src/lib.rs:13-318`, `crates/ullm-metal/src/forward.rs:24-110, 230-760`) under the
//! same names, over the C ABI of `libullm_cuda` (`include/ullm_cuda.h`).  `ullm-model` switches
//! backends by changing one `use` line (`crates/ullm-model/src/lib.rs:20`) and one dependency
//! (`crates/ullm-model/Cargo.toml:15`).
//!
//! Not compiled in the repository that carries it (no Rust toolchain there); `src/ffi.rs` is
//! generated from the C headers by `gen_ffi.py`, and a test of that repository keeps the two equal.
//!
//! There is no CPU fallback: without a B200 `CudaContext::new` / `GpuForward::new` return
//! `Error::Unsupported("no CUDA device available")`, as `MetalContext::new` does without a Metal
//! device (`crates/ullm-metal/src/lib.rs:31-33`).

pub mod ffi;

use std::ffi::CStr;
use std::os::raw::c_int;
use std::ptr;

use ullm_core::{DType, Error, Result};

// ---------------------------------------------------------------------------
// The six input types ullm-model imports, field for field as in forward.rs:24-110
// ---------------------------------------------------------------------------

/// Scalar hyperparameters and architecture toggles (forward.rs:24-51).
#[derive(Debug, Clone, Copy)]
pub struct GpuParams {
    pub n_embd: usize,
    pub n_layer: usize,
    pub n_head: usize,
    pub n_kv_head: usize,
    pub head_dim: usize,
    pub n_ff: usize,
    pub n_ctx: usize,
    pub vocab: usize,
    pub rope_theta: f32,
    pub eps: f32,
    pub rope_neox: bool,
    pub qk_norm: bool,
    pub sandwich_norm: bool,
    pub geglu: bool,
    pub n_experts: usize,
    pub n_experts_used: usize,
    pub moe_inter: usize,
    pub sliding_window: usize,
}

/// A weight matrix to upload (forward.rs:56-64).
pub struct GpuWeight<'a> {
    pub dtype: DType,
    pub bytes: &'a [u8],
    pub out: usize,
    pub cols: usize,
    pub mlx_scales: Option<&'a [f32]>,
    pub mlx_biases: Option<&'a [f32]>,
    pub mlx_group: usize,
}

/// Stacked per-expert MLX 4-bit weights (forward.rs:67-75).
pub struct GpuExperts {
    pub bytes: Vec<u8>,
    pub scales: Vec<f32>,
    pub biases: Vec<f32>,
    pub n_experts: usize,
    pub out: usize,
    pub cols: usize,
    pub group: usize,
}

/// Per-layer weights (forward.rs:78-100).
pub struct GpuLayerInput<'a> {
    pub attn_norm: &'a [f32],
    pub wq: GpuWeight<'a>,
    pub wk: GpuWeight<'a>,
    pub wv: GpuWeight<'a>,
    pub wo: GpuWeight<'a>,
    pub q_bias: Option<&'a [f32]>,
    pub k_bias: Option<&'a [f32]>,
    pub v_bias: Option<&'a [f32]>,
    pub q_norm: Option<&'a [f32]>,
    pub k_norm: Option<&'a [f32]>,
    pub post_attn_norm: Option<&'a [f32]>,
    pub post_ffn_norm: Option<&'a [f32]>,
    pub ffn_norm: &'a [f32],
    pub w_gate: GpuWeight<'a>,
    pub w_up: GpuWeight<'a>,
    pub w_down: GpuWeight<'a>,
    pub moe_gate: Option<GpuWeight<'a>>,
    pub experts_gate: Option<GpuExperts>,
    pub experts_up: Option<GpuExperts>,
    pub experts_down: Option<GpuExperts>,
}

/// The whole model (forward.rs:105-110).
pub struct GpuModelInput<'a> {
    pub params: GpuParams,
    pub output: GpuWeight<'a>,
    pub final_norm: &'a [f32],
    pub layers: Vec<GpuLayerInput<'a>>,
}

// ---------------------------------------------------------------------------
// helpers
// ---------------------------------------------------------------------------

/// ggml tensor type ids (crates/ullm-gguf/src/types.rs:7-29) plus the library's id for MLX words.
fn dtype_id(d: DType) -> Result<c_int> {
    Ok(match d {
        DType::F32 => ffi::ULLM_DTYPE_F32,
        DType::F16 => ffi::ULLM_DTYPE_F16,
        DType::BF16 => ffi::ULLM_DTYPE_BF16,
        DType::Q4K => ffi::ULLM_DTYPE_Q4_K,
        DType::Q6K => ffi::ULLM_DTYPE_Q6_K,
        DType::U32 => ffi::ULLM_DTYPE_MLX_U32,
        other => return Err(Error::Unsupported(format!("no CUDA kernel for {other:?} yet"))),
    })
}

/// UNSUPPORTED -> `Error::Unsupported`, everything else -> `Error::Format` (crates/ullm-core/src/error.rs:11-20).
fn check(rc: c_int, ctx: *const ffi::ullm_cuda_ctx) -> Result<()> {
    if rc == ffi::ULLM_OK {
        return Ok(());
    }
    let msg = if ctx.is_null() {
        String::from("libullm_cuda call failed")
    } else {
        unsafe { CStr::from_ptr(ffi::ullm_cuda_last_error(ctx)) }.to_string_lossy().into_owned()
    };
    Err(if rc == ffi::ULLM_ERR_UNSUPPORTED { Error::Unsupported(msg) } else { Error::Format(format!("{msg} (status {rc})")) })
}

fn opt_ptr(v: Option<&[f32]>) -> *const f32 {
    v.map_or(ptr::null(), |s| s.as_ptr())
}

fn c_weight(w: &GpuWeight) -> Result<ffi::ullm_gpu_weight> {
    Ok(ffi::ullm_gpu_weight {
        dtype: dtype_id(w.dtype)?,
        bytes: w.bytes.as_ptr().cast(),
        len: w.bytes.len(),
        out: w.out,
        cols: w.cols,
        mlx_scales: opt_ptr(w.mlx_scales),
        mlx_biases: opt_ptr(w.mlx_biases),
        mlx_group: w.mlx_group,
    })
}

fn empty_weight() -> ffi::ullm_gpu_weight {
    ffi::ullm_gpu_weight { dtype: 0, bytes: ptr::null(), len: 0, out: 0, cols: 0, mlx_scales: ptr::null(), mlx_biases: ptr::null(), mlx_group: 0 }
}

// ---------------------------------------------------------------------------
// CudaContext: the method set of MetalContext (crates/ullm-metal/src/lib.rs:18-318)
// ---------------------------------------------------------------------------

/// A resident device buffer (`metal::Buffer` in the reference surface).
pub struct Buffer {
    ctx: *mut ffi::ullm_cuda_ctx,
    raw: *mut ffi::ullm_cuda_buf,
}
impl Drop for Buffer {
    fn drop(&mut self) {
        unsafe { ffi::ullm_cuda_buf_free(self.ctx, self.raw) }
    }
}

pub struct CudaContext {
    raw: *mut ffi::ullm_cuda_ctx,
}
// Same invariant as the reference states for its GPU objects (forward.rs:221-225): may move between
// threads, never used by two at once.
unsafe impl Send for CudaContext {}

impl CudaContext {
    /// `MetalContext::new` (lib.rs:31): device 0.
    pub fn new() -> Result<Self> {
        Self::on_device(0)
    }
    pub fn on_device(device: i32) -> Result<Self> {
        let mut raw = ptr::null_mut();
        match unsafe { ffi::ullm_cuda_ctx_create(device, &mut raw) } {
            ffi::ULLM_OK => Ok(Self { raw }),
            ffi::ULLM_ERR_UNSUPPORTED => Err(Error::Unsupported("no CUDA device available".into())),
            rc => Err(Error::Format(format!("CUDA context creation failed (status {rc})"))),
        }
    }
    pub fn device_name(&self) -> String {
        let mut buf = [0 as std::os::raw::c_char; 256];
        unsafe { ffi::ullm_cuda_device_name(self.raw, buf.as_mut_ptr(), buf.len()) };
        unsafe { CStr::from_ptr(buf.as_ptr()) }.to_string_lossy().into_owned()
    }
    /// `upload` (lib.rs:64).  The reference cannot fail here; an allocation failure panics like its `expect`s.
    pub fn upload(&self, bytes: &[u8]) -> Buffer {
        let mut raw = ptr::null_mut();
        let rc = unsafe { ffi::ullm_cuda_upload(self.raw, bytes.as_ptr().cast(), bytes.len(), &mut raw) };
        check(rc, self.raw).expect("device upload");
        Buffer { ctx: self.raw, raw }
    }
    /// `matvec_quant` (lib.rs:83-94).
    pub fn matvec_quant(&self, dtype: DType, w_bytes: &[u8], x: &[f32], out_dim: usize, in_dim: usize) -> Result<Vec<f32>> {
        let mut y = vec![0.0f32; out_dim];
        let rc = unsafe {
            ffi::ullm_cuda_matvec_quant(self.raw, dtype_id(dtype)?, w_bytes.as_ptr().cast(), w_bytes.len(), x.as_ptr(), y.as_mut_ptr(), out_dim, in_dim)
        };
        check(rc, self.raw).map(|_| y)
    }
    /// `matvec_resident` (lib.rs:97-107).
    pub fn matvec_resident(&self, dtype: DType, wbuf: &Buffer, x: &[f32], out_dim: usize, in_dim: usize) -> Result<Vec<f32>> {
        let mut y = vec![0.0f32; out_dim];
        let rc = unsafe { ffi::ullm_cuda_matvec_resident(self.raw, dtype_id(dtype)?, wbuf.raw, x.as_ptr(), y.as_mut_ptr(), out_dim, in_dim) };
        check(rc, self.raw).map(|_| y)
    }
    /// `matvec_mlx4` (lib.rs:112-158): infallible in the reference, so a failure panics.
    #[allow(clippy::too_many_arguments)]
    pub fn matvec_mlx4(&self, w: &[u8], scales: &[f32], biases: &[f32], x: &[f32], out_dim: usize, in_dim: usize, group_size: usize) -> Vec<f32> {
        let mut y = vec![0.0f32; out_dim];
        let rc = unsafe {
            ffi::ullm_cuda_matvec_mlx4(self.raw, w.as_ptr().cast(), scales.as_ptr(), biases.as_ptr(), x.as_ptr(), y.as_mut_ptr(), out_dim, in_dim, group_size)
        };
        check(rc, self.raw).expect("matvec_mlx4");
        y
    }
    /// `matmul_mlx4` (lib.rs:212-266): activations and outputs token-major.
    #[allow(clippy::too_many_arguments)]
    pub fn matmul_mlx4(&self, w: &[u8], scales: &[f32], biases: &[f32], x: &[f32], out_dim: usize, in_dim: usize, group_size: usize, s: usize) -> Vec<f32> {
        let mut y = vec![0.0f32; s * out_dim];
        let rc = unsafe {
            ffi::ullm_cuda_matmul_mlx4(self.raw, w.as_ptr().cast(), scales.as_ptr(), biases.as_ptr(), x.as_ptr(), y.as_mut_ptr(), out_dim, in_dim, group_size, s)
        };
        check(rc, self.raw).expect("matmul_mlx4");
        y
    }
    /// Quantized prefill product (`GpuForward::matmul`, forward.rs:679-725) on host bytes.
    pub fn matmul_quant(&self, dtype: DType, w_bytes: &[u8], x: &[f32], out_dim: usize, in_dim: usize, s: usize) -> Result<Vec<f32>> {
        let mut y = vec![0.0f32; s * out_dim];
        let rc = unsafe {
            ffi::ullm_cuda_matmul_quant(self.raw, dtype_id(dtype)?, w_bytes.as_ptr().cast(), w_bytes.len(), x.as_ptr(), y.as_mut_ptr(), out_dim, in_dim, s)
        };
        check(rc, self.raw).map(|_| y)
    }
    /// Dense f32 / bf16 products (`matvec`, `matmul_bf16`, lib.rs:73, :163) serve the reference's `metal-check`
    /// command only and lie outside the quantized path this backend accelerates.
    pub fn matvec(&self, _w: &[f32], _x: &[f32], _out_dim: usize, _in_dim: usize) -> Vec<f32> {
        panic!("ullm-cuda: the dense f32 matvec is not built (quantized weights only)")
    }
    pub fn matmul_bf16(&self, _w: &[u8], _x: &[f32], _out_dim: usize, _in_dim: usize, _s: usize) -> Vec<f32> {
        panic!("ullm-cuda: the dense bf16 matmul is not built (quantized weights only)")
    }
}
impl Drop for CudaContext {
    fn drop(&mut self) {
        unsafe { ffi::ullm_cuda_ctx_destroy(self.raw) }
    }
}

// ---------------------------------------------------------------------------
// GpuForward (forward.rs:162-760)
// ---------------------------------------------------------------------------

/// One op of `forward_debug`'s report: non-finite counts and the largest finite magnitude.
#[derive(Debug, Clone)]
pub struct DebugStat {
    pub label: String,
    pub nan: u64,
    pub inf: u64,
    pub maxabs: f32,
}

/// The resident decode engine: weights, KV cache and activations live on the GPU; one submission per token.
pub struct GpuForward {
    ctx: CudaContext,
    raw: *mut ffi::ullm_cuda_fwd,
    vocab: usize,
    n_embd: usize,
}
unsafe impl Send for GpuForward {} // forward.rs:221-225: never concurrent work on one instance

fn c_experts(g: &GpuExperts, u: &GpuExperts, d: &GpuExperts) -> ffi::ullm_moe_experts_input {
    // gate / up: [n_experts, inter, hidden / 8] words; down: [n_experts, hidden, inter / 8] (forward.rs:67-75)
    ffi::ullm_moe_experts_input {
        gate_w: g.bytes.as_ptr().cast(),
        gate_scales: g.scales.as_ptr().cast(),
        gate_biases: g.biases.as_ptr().cast(),
        up_w: u.bytes.as_ptr().cast(),
        up_scales: u.scales.as_ptr().cast(),
        up_biases: u.biases.as_ptr().cast(),
        down_w: d.bytes.as_ptr().cast(),
        down_scales: d.scales.as_ptr().cast(),
        down_biases: d.biases.as_ptr().cast(),
        table_dtype: ffi::ULLM_DTYPE_F32, // the reference hands the tables over widened to f32 (lib.rs:751-771)
        n_experts: g.n_experts,
        hidden: g.cols,
        inter: g.out,
        group: g.group,
    }
}

impl GpuForward {
    /// `GpuForward::new` (forward.rs:230): copies everything into device memory; the input is borrowed for the call.
    pub fn new(input: &GpuModelInput) -> Result<Self> {
        let ctx = CudaContext::new()?;
        let p = &input.params;
        let params = ffi::ullm_gpu_params {
            n_embd: p.n_embd,
            n_layer: p.n_layer,
            n_head: p.n_head,
            n_kv_head: p.n_kv_head,
            head_dim: p.head_dim,
            n_ff: p.n_ff,
            n_ctx: p.n_ctx,
            vocab: p.vocab,
            rope_theta: p.rope_theta,
            eps: p.eps,
            rope_neox: p.rope_neox as c_int,
            qk_norm: p.qk_norm as c_int,
            sandwich_norm: p.sandwich_norm as c_int,
            geglu: p.geglu as c_int,
            n_experts: p.n_experts,
            n_experts_used: p.n_experts_used,
            moe_inter: p.moe_inter,
            sliding_window: p.sliding_window,
            kv_f16: 0, // the reference keeps an f32 KV cache (forward.rs:355-356)
        };
        // the experts' descriptions must outlive the call: one slot per layer
        let mut experts: Vec<Option<ffi::ullm_moe_experts_input>> = Vec::with_capacity(input.layers.len());
        for l in &input.layers {
            experts.push(match (&l.experts_gate, &l.experts_up, &l.experts_down) {
                (Some(g), Some(u), Some(d)) => Some(c_experts(g, u, d)),
                _ => None,
            });
        }
        let mut layers = Vec::with_capacity(input.layers.len());
        for (l, x) in input.layers.iter().zip(experts.iter()) {
            if l.post_attn_norm.is_some() || l.post_ffn_norm.is_some() {
                return Err(Error::Unsupported("sandwich norms are not built".into()));
            }
            layers.push(ffi::ullm_gpu_layer_input {
                attn_norm: l.attn_norm.as_ptr(),
                ffn_norm: l.ffn_norm.as_ptr(),
                wq: c_weight(&l.wq)?,
                wk: c_weight(&l.wk)?,
                wv: c_weight(&l.wv)?,
                wo: c_weight(&l.wo)?,
                w_gate: if x.is_some() { empty_weight() } else { c_weight(&l.w_gate)? },
                w_up: if x.is_some() { empty_weight() } else { c_weight(&l.w_up)? },
                w_down: if x.is_some() { empty_weight() } else { c_weight(&l.w_down)? },
                q_bias: opt_ptr(l.q_bias),
                k_bias: opt_ptr(l.k_bias),
                v_bias: opt_ptr(l.v_bias),
                q_norm: opt_ptr(l.q_norm),
                k_norm: opt_ptr(l.k_norm),
                moe_gate: match &l.moe_gate {
                    Some(w) => c_weight(w)?,
                    None => empty_weight(),
                },
                experts: x.as_ref().map_or(ptr::null(), |e| e as *const _),
            });
        }
        let model = ffi::ullm_gpu_model_input {
            params,
            output: c_weight(&input.output)?,
            final_norm: input.final_norm.as_ptr(),
            layers: layers.as_ptr(),
            mlx_table_dtype: ffi::ULLM_DTYPE_F32,
        };
        let mut raw = ptr::null_mut();
        let rc = unsafe { ffi::ullm_cuda_forward_create(ctx.raw, &model, &mut raw) };
        check(rc, ctx.raw)?;
        Ok(Self { ctx, raw, vocab: p.vocab, n_embd: p.n_embd })
    }

    /// `forward` (forward.rs:384): one token at `pos`; returns the vocab logits.
    pub fn forward(&self, x_init: &[f32], pos: usize) -> Result<Vec<f32>> {
        assert_eq!(x_init.len(), self.n_embd);
        let mut logits = vec![0.0f32; self.vocab];
        let rc = unsafe { ffi::ullm_cuda_forward(self.raw, x_init.as_ptr(), pos, logits.as_mut_ptr()) };
        check(rc, self.ctx.raw).map(|_| logits)
    }

    /// `supports_batched_prefill` (forward.rs:744).
    pub fn supports_batched_prefill(&self) -> bool {
        unsafe { ffi::ullm_cuda_forward_supports_batched_prefill(self.raw) != 0 }
    }

    /// `forward_batch` (forward.rs:757): `embeds` is `[s, n_embd]` token-major for positions 0..s-1.
    pub fn forward_batch(&self, embeds: &[f32], s: usize) -> Result<Vec<f32>> {
        assert_eq!(embeds.len(), s * self.n_embd);
        let mut logits = vec![0.0f32; self.vocab];
        let rc = unsafe { ffi::ullm_cuda_forward_batch(self.raw, embeds.as_ptr(), s, logits.as_mut_ptr()) };
        check(rc, self.ctx.raw).map(|_| logits)
    }

    /// The numbers behind `forward_debug`: layer 0 one op at a time.
    pub fn forward_debug_stats(&self, x_init: &[f32], pos: usize) -> Result<Vec<DebugStat>> {
        let mut raw = vec![ffi::ullm_debug_stat { label: [0; 16], nan: 0, inf: 0, maxabs: 0.0 }; 32];
        let mut n = 0usize;
        let rc = unsafe { ffi::ullm_cuda_forward_debug(self.raw, x_init.as_ptr(), pos, raw.as_mut_ptr(), raw.len(), &mut n) };
        check(rc, self.ctx.raw)?;
        Ok(raw[..n]
            .iter()
            .map(|s| DebugStat {
                label: unsafe { CStr::from_ptr(s.label.as_ptr()) }.to_string_lossy().into_owned(),
                nan: s.nan,
                inf: s.inf,
                maxabs: s.maxabs,
            })
            .collect())
    }

    /// `forward_debug` (forward.rs:530-635): prints one line per op of layer 0, in the reference's format.
    pub fn forward_debug(&self, x_init: &[f32], pos: usize) {
        match self.forward_debug_stats(x_init, pos) {
            Ok(stats) => {
                for s in stats {
                    eprintln!("[dbg pos{pos}] {:<14} nan={} inf={} maxabs={:.4}", s.label, s.nan, s.inf, s.maxabs);
                }
            }
            Err(e) => eprintln!("[dbg pos{pos}] unavailable: {e}"),
        }
    }
}
impl Drop for GpuForward {
    fn drop(&mut self) {
        unsafe { ffi::ullm_cuda_forward_destroy(self.raw) }
    }
}

// ---------------------------------------------------------------------------
// Row-sharded matrices over the GPUs of one node (no counterpart in ullm-metal; the reference's
// roadmap lists multi-device scale-out as open, docs/roadmap.md:83).  The split is the one the CPU
// path already uses: output rows are independent (crates/ullm-model/src/math.rs:11-21).
// ---------------------------------------------------------------------------

/// One rank's end of a group of `world` GPUs: a gather buffer of `y_floats` floats with the same
/// layout on every rank, in which the caller places full-length result vectors by offset.
pub struct ShardGroup {
    ctx: *mut ffi::ullm_cuda_ctx,
    raw: *mut ffi::ullm_cuda_shard,
    world: usize,
    rank: usize,
}
unsafe impl Send for ShardGroup {}

/// This rank's rows of a matrix, resident on its GPU.
pub struct ShardedWeight {
    ctx: *mut ffi::ullm_cuda_ctx,
    raw: *mut ffi::ullm_cuda_weight,
    pub out_total: usize,
    pub cols: usize,
}
impl Drop for ShardedWeight {
    fn drop(&mut self) {
        unsafe { ffi::ullm_cuda_weight_destroy(self.ctx, self.raw) }
    }
}

/// One matvec of a step: `y[y_offset .. y_offset + out_total] = W x` in every rank's gather buffer.
pub struct ShardOp<'a> {
    pub w: &'a ShardedWeight,
    /// this rank's copy of the whole input vector, on the device
    pub x: &'a Buffer,
    pub y_offset: usize,
}

impl ShardGroup {
    pub fn new(ctx: &CudaContext, world: usize, rank: usize, y_floats: usize) -> Result<Self> {
        let mut raw = ptr::null_mut();
        check(unsafe { ffi::ullm_cuda_shard_create(ctx.raw, world as c_int, rank as c_int, y_floats, &mut raw) }, ctx.raw)?;
        Ok(Self { ctx: ctx.raw, raw, world, rank })
    }
    /// The bytes the other ranks' processes need to reach this rank's buffer (plain data: send them by any means).
    pub fn export(&self) -> Result<[u8; ffi::ULLM_SHARD_HANDLE_BYTES]> {
        let mut h = [0u8; ffi::ULLM_SHARD_HANDLE_BYTES];
        check(unsafe { ffi::ullm_cuda_shard_export(self.raw, h.as_mut_ptr().cast()) }, self.ctx)?;
        Ok(h)
    }
    /// `handles`: every rank's `export()`, in rank order.  All ranks connect before any runs a step.
    pub fn connect(&mut self, handles: &[[u8; ffi::ULLM_SHARD_HANDLE_BYTES]]) -> Result<()> {
        if handles.len() != self.world {
            return Err(Error::Format(format!("need {} handles, got {}", self.world, handles.len())));
        }
        check(unsafe { ffi::ullm_cuda_shard_connect(self.raw, handles.as_ptr().cast()) }, self.ctx)
    }
    pub fn rank(&self) -> usize {
        self.rank
    }
    /// Uploads this rank's rows of `full` (a description of the WHOLE matrix).
    pub fn weight(&self, full: &GpuWeight) -> Result<ShardedWeight> {
        let cw = c_weight(full)?;
        let mut raw = ptr::null_mut();
        check(unsafe { ffi::ullm_cuda_shard_weight_create(self.raw, &cw, ffi::ULLM_DTYPE_F32, &mut raw) }, self.ctx)?;
        Ok(ShardedWeight { ctx: self.ctx, raw, out_total: full.out, cols: full.cols })
    }
    /// One step: every op's rows are computed here and stored into every rank's gather buffer; returns
    /// (in stream order) when every rank's rows are in this rank's buffer.  A rank that does not answer within
    /// the context's limit ends the step with an error instead of a hang.  Every rank runs the same steps.
    pub fn matvec(&self, ops: &[ShardOp]) -> Result<()> {
        let c: Vec<ffi::ullm_shard_op> = ops
            .iter()
            .map(|o| ffi::ullm_shard_op { w: o.w.raw, d_x: unsafe { ffi::ullm_cuda_buf_ptr(o.x.raw) }.cast(), y_offset: o.y_offset, row0: 0 })
            .collect();
        check(unsafe { ffi::ullm_cuda_shard_matvec_dev(self.raw, c.len(), c.as_ptr(), 0, ptr::null_mut()) }, self.ctx)
    }
    /// `n` gathered floats at `offset` of this rank's buffer (waits for the context's stream).
    pub fn read(&self, offset: usize, n: usize) -> Result<Vec<f32>> {
        let mut v = vec![0f32; n];
        check(unsafe { ffi::ullm_cuda_shard_read(self.raw, offset, v.as_mut_ptr(), n) }, self.ctx)?;
        Ok(v)
    }
    /// After a time-out the ranks are out of step: every rank resets, with a barrier of the caller's in between.
    pub fn reset(&mut self) -> Result<()> {
        check(unsafe { ffi::ullm_cuda_shard_reset(self.raw) }, self.ctx)
    }
}
impl Drop for ShardGroup {
    fn drop(&mut self) {
        unsafe { ffi::ullm_cuda_shard_destroy(self.raw) }
    }
}
