//! NOT COMPILED IN THIS ENVIRONMENT (the build image has no Rust toolchain): written against
//! candle-core / candle-nn 0.8.3 by reading their sources, to be reviewed and compiled by a maintainer.
//!
//! candle front ends for the B200 norm + embedding kernels.  Each op keeps candle's `CustomOp`
//! contract -- same name, same checks, same error strings, a CPU path with candle's arithmetic -- and
//! its `cuda_fwd` allocates the output as candle does and hands raw device pointers to the C ABI
//! (`ffi.rs`), the way candle-flash-attn/src/lib.rs:141-208 does for `run_mha`.
//!
//! | here                                | replaces in candle                                             |
//! |-------------------------------------|----------------------------------------------------------------|
//! | `RmsNorm: CustomOp2`, `rms_norm`    | candle-nn/src/ops.rs:437-652                                   |
//! | `LayerNorm: CustomOp3`, `layer_norm`| candle-nn/src/ops.rs:654-909                                   |
//! | `rms_norm_slow`, `layer_norm_slow`  | candle-nn/src/ops.rs:628-639, 876-894 (one launch, not eight)  |
//! | `SoftmaxLastDim: CustomOp1`         | candle-nn/src/ops.rs:289-435                                   |
//! | `Rope: CustomOp3`                   | candle-nn/src/rotary_emb.rs (rope_i, rope, rope_thd)           |
//! | `index_select`                      | candle-core/src/cuda_backend/mod.rs:352-410, 1622-1626         |
//! | `QEmbedding: CustomOp1`             | new: lookup out of GGML blocks (cf. quantized/mod.rs:464-525)  |
pub mod ffi;

use candle::backend::BackendStorage;
use candle::cuda_backend::cudarc::driver::{DevicePtr, DeviceSlice};
use candle::cuda_backend::WrapErr;
use candle::{CpuStorage, CudaDevice, CudaStorage, DType, Layout, Result, Shape, Tensor, WithDType};
use core::ffi::{c_int, c_void};
use half::{bf16, f16};
use rayon::prelude::*;

fn check(rc: c_int) -> Result<()> {
    if rc == 0 {
        return Ok(());
    }
    let msg = unsafe { std::ffi::CStr::from_ptr(ffi::cb200_last_error()) };
    candle::bail!("{}", msg.to_string_lossy())
}

fn dtype_code(dtype: DType, op: &str) -> Result<c_int> {
    match dtype {
        DType::F32 => Ok(ffi::DTYPE_F32),
        DType::F16 => Ok(ffi::DTYPE_F16),
        DType::BF16 => Ok(ffi::DTYPE_BF16),
        d => candle::bail!("unsupported dtype for {op} {d:?}"),
    }
}

fn stream(dev: &CudaDevice) -> *mut c_void {
    // the CUstream candle enqueues its own kernels on (cudarc's device stream)
    *dev.cu_stream() as *mut c_void
}

/// Device address of the first element of a contiguous tensor: slice base + start offset, as
/// `src.slice(o1..o2)` does in candle-nn/src/ops.rs:536-543.
fn base_ptr(storage: &CudaStorage, layout: &Layout, what: &str) -> Result<*const c_void> {
    let (o1, _o2) = match layout.contiguous_offsets() {
        None => candle::bail!("{what} has to be contiguous"),
        Some(o) => o,
    };
    let esz = storage.dtype().size_in_bytes();
    let base = match storage.dtype() {
        DType::F32 => *storage.as_cuda_slice::<f32>()?.device_ptr(),
        DType::F16 => *storage.as_cuda_slice::<f16>()?.device_ptr(),
        DType::BF16 => *storage.as_cuda_slice::<bf16>()?.device_ptr(),
        DType::U8 => *storage.as_cuda_slice::<u8>()?.device_ptr(),
        DType::U32 => *storage.as_cuda_slice::<u32>()?.device_ptr(),
        DType::I64 => *storage.as_cuda_slice::<i64>()?.device_ptr(),
        d => candle::bail!("unsupported dtype {d:?}"),
    };
    Ok((base + (o1 * esz) as u64) as *const c_void)
}

/// Uninitialised output of `el` elements of `dtype` (candle: `unsafe { dev.alloc::<T>(el) }`,
/// candle-nn/src/ops.rs:557); the kernels write every element.
fn alloc_like(dev: &CudaDevice, dtype: DType, el: usize) -> Result<(CudaStorage, *mut c_void)> {
    macro_rules! alloc {
        ($t:ty) => {{
            let slice = unsafe { dev.alloc::<$t>(el) }.w()?;
            let ptr = *slice.device_ptr() as *mut c_void;
            (CudaStorage::wrap_cuda_slice(slice, dev.clone()), ptr)
        }};
    }
    Ok(match dtype {
        DType::F32 => alloc!(f32),
        DType::F16 => alloc!(f16),
        DType::BF16 => alloc!(bf16),
        d => candle::bail!("unsupported dtype {d:?}"),
    })
}

// ---------------------------------------------------------------------------------------------
// CPU arithmetic (what `cpu_fwd` must keep computing): every row sum strictly left to right in f32,
// the roundings where candle's CPU backend has them.
// ---------------------------------------------------------------------------------------------
fn cpu_rms_norm<T: WithDType + num_like::FloatLike>(src: &[T], alpha: &[T], cols: usize, eps: f32) -> Vec<T> {
    let mut dst = vec![T::zero(); src.len()];
    src.par_chunks(cols).zip(dst.par_chunks_mut(cols)).for_each(|(s, d)| {
        let mut sum2 = 0f32;
        for v in s {
            let v = v.to_f32();
            sum2 += v * v;
        }
        let m = T::from_f32((sum2 / cols as f32 + eps).sqrt());
        for ((d, s), a) in d.iter_mut().zip(s).zip(alpha) {
            *d = *s / m * *a
        }
    });
    dst
}

fn cpu_layer_norm<T: WithDType + num_like::FloatLike>(src: &[T], alpha: &[T], beta: &[T], cols: usize, eps: f32) -> Vec<T> {
    let mut dst = vec![T::zero(); src.len()];
    src.par_chunks(cols).zip(dst.par_chunks_mut(cols)).for_each(|(s, d)| {
        let (mut sum, mut sum2) = (0f32, 0f32);
        for v in s {
            let v = v.to_f32();
            sum += v;
            sum2 += v * v;
        }
        let mean = sum / cols as f32;
        let var = sum2 / cols as f32 - mean * mean;
        let inv_std = (var + eps).sqrt().recip();
        for ((d, s), (a, b)) in d.iter_mut().zip(s).zip(alpha.iter().zip(beta)) {
            *d = T::from_f32((s.to_f32() - mean) * inv_std * a.to_f32() + b.to_f32())
        }
    });
    dst
}

/// The float element types of this path, with the conversions the loops above need.
mod num_like {
    use half::{bf16, f16};
    pub trait FloatLike: Copy + Send + Sync + std::ops::Div<Output = Self> + std::ops::Mul<Output = Self> {
        fn zero() -> Self;
        fn to_f32(self) -> f32;
        fn from_f32(v: f32) -> Self;
    }
    macro_rules! imp {
        ($t:ty, $z:expr, $to:expr, $from:expr) => {
            impl FloatLike for $t {
                fn zero() -> Self { $z }
                fn to_f32(self) -> f32 { $to(self) }
                fn from_f32(v: f32) -> Self { $from(v) }
            }
        };
    }
    imp!(f32, 0f32, |v| v, |v| v);
    imp!(f16, f16::ZERO, f16::to_f32, f16::from_f32);
    imp!(bf16, bf16::ZERO, bf16::to_f32, bf16::from_f32);
}

fn contiguous<'a, T>(s: &'a [T], l: &Layout, what: &str) -> Result<&'a [T]> {
    match l.contiguous_offsets() {
        None => candle::bail!("{what} has to be contiguous"),
        Some((o1, o2)) => Ok(&s[o1..o2]),
    }
}

// ---------------------------------------------------------------------------------------------
// rms_norm
// ---------------------------------------------------------------------------------------------
#[derive(Debug, Clone)]
pub struct RmsNorm {
    pub eps: f32,
}

impl candle::CustomOp2 for RmsNorm {
    fn name(&self) -> &'static str {
        "rms-norm"
    }

    fn cpu_fwd(&self, s1: &CpuStorage, l1: &Layout, s2: &CpuStorage, l2: &Layout) -> Result<(CpuStorage, Shape)> {
        let cols = *l1.dims().last().ok_or_else(|| candle::Error::msg("unexpected rank, expected: at least 1, got: 0"))?;
        use CpuStorage as C;
        let out = match (s1, s2) {
            (C::F32(x), C::F32(a)) => C::F32(cpu_rms_norm(contiguous(x, l1, "input")?, contiguous(a, l2, "alpha")?, cols, self.eps)),
            (C::F16(x), C::F16(a)) => C::F16(cpu_rms_norm(contiguous(x, l1, "input")?, contiguous(a, l2, "alpha")?, cols, self.eps)),
            (C::BF16(x), C::BF16(a)) => C::BF16(cpu_rms_norm(contiguous(x, l1, "input")?, contiguous(a, l2, "alpha")?, cols, self.eps)),
            _ => candle::bail!("unsupported dtype for rmsnorm {:?}", s1.dtype()),
        };
        Ok((out, l1.shape().clone()))
    }

    fn cuda_fwd(&self, s1: &CudaStorage, l1: &Layout, s2: &CudaStorage, l2: &Layout) -> Result<(CudaStorage, Shape)> {
        let dt = dtype_code(s1.dtype(), "rmsnorm")?;
        if s2.dtype() != s1.dtype() {
            candle::bail!("unsupported dtype for rmsnorm {:?}", s1.dtype())
        }
        let x = base_ptr(s1, l1, "input")?;
        let alpha = base_ptr(s2, l2, "alpha")?;
        let el = l1.shape().elem_count();
        let cols = *l1.dims().last().unwrap();
        let rows = if cols == 0 { 0 } else { el / cols };
        let dev = s1.device();
        let (dst, y) = alloc_like(dev, s1.dtype(), el)?;
        check(unsafe {
            ffi::cb200_rms_norm(x, std::ptr::null(), alpha, y, std::ptr::null_mut(), rows as i64, cols as i32, self.eps, dt,
                                0, stream(dev))
        })?;
        Ok((dst, l1.shape().clone()))
    }
}

/// `candle_nn::ops::rms_norm(xs, alpha, eps)` (candle-nn/src/ops.rs:641-652).
pub fn rms_norm(xs: &Tensor, alpha: &Tensor, eps: f32) -> Result<Tensor> {
    let hidden_size_xs = xs.dim(candle::D::Minus1)?;
    let hidden_size_alpha = alpha.dims1()?;
    if hidden_size_xs != hidden_size_alpha {
        candle::bail!("shape mismatch in rms-norm {:?} {:?}", xs.shape(), alpha.shape())
    }
    xs.apply_op2_no_bwd(alpha, &RmsNorm { eps })
}

/// `(xs + residual)` followed by `rms_norm`, fused: returns `(y, xs + residual)`.  Replaces
/// `let x = (attn + residual)?; rms.forward(&x)` in candle-transformers/src/models/llama.rs:446-450.
/// CUDA only; on other devices compose the two ops.
pub fn rms_norm_residual(xs: &Tensor, residual: &Tensor, alpha: &Tensor, eps: f32) -> Result<(Tensor, Tensor)> {
    if !xs.device().is_cuda() {
        let h = (xs + residual)?;
        return Ok((rms_norm(&h, alpha, eps)?, h));
    }
    if xs.shape() != residual.shape() || xs.dtype() != residual.dtype() {
        candle::bail!("shape mismatch in binary op add, lhs: {:?}, rhs: {:?}", xs.shape(), residual.shape())
    }
    let h = xs.zeros_like()?; // receives xs + residual
    let y = xs.zeros_like()?;
    // Pointers are taken from the storages directly: four tensors do not fit a CustomOp3.
    let dt = dtype_code(xs.dtype(), "rmsnorm")?;
    let cols = xs.dim(candle::D::Minus1)?;
    let rows = xs.elem_count() / cols.max(1);
    let ptr = |t: &Tensor, what: &str| -> Result<(*const c_void, CudaDevice)> {
        let (st, l) = t.storage_and_layout();
        match &*st {
            candle::Storage::Cuda(c) => Ok((base_ptr(c, l, what)?, c.device().clone())),
            _ => candle::bail!("rms_norm_residual expects cuda tensors"),
        }
    };
    let (x, dev) = ptr(xs, "input")?;
    let (r, _) = ptr(residual, "input")?;
    let (a, _) = ptr(alpha, "alpha")?;
    let (yp, _) = ptr(&y, "output")?;
    let (hp, _) = ptr(&h, "output")?;
    check(unsafe {
        ffi::cb200_rms_norm(x, r, a, yp as *mut c_void, hp as *mut c_void, rows as i64, cols as i32, eps, dt, 0, stream(&dev))
    })?;
    Ok((y, h))
}

// ---------------------------------------------------------------------------------------------
// layer_norm
// ---------------------------------------------------------------------------------------------
#[derive(Debug, Clone)]
pub struct LayerNorm {
    pub eps: f32,
}

impl candle::CustomOp3 for LayerNorm {
    fn name(&self) -> &'static str {
        "layer-norm"
    }

    fn cpu_fwd(&self, s1: &CpuStorage, l1: &Layout, s2: &CpuStorage, l2: &Layout, s3: &CpuStorage, l3: &Layout)
        -> Result<(CpuStorage, Shape)> {
        let cols = *l1.dims().last().ok_or_else(|| candle::Error::msg("unexpected rank, expected: at least 1, got: 0"))?;
        use CpuStorage as C;
        macro_rules! run {
            ($v:ident, $x:expr, $a:expr, $b:expr) => {
                C::$v(cpu_layer_norm(contiguous($x, l1, "input")?, contiguous($a, l2, "alpha")?, contiguous($b, l3, "beta")?, cols, self.eps))
            };
        }
        let out = match (s1, s2, s3) {
            (C::F32(x), C::F32(a), C::F32(b)) => run!(F32, x, a, b),
            (C::F16(x), C::F16(a), C::F16(b)) => run!(F16, x, a, b),
            (C::BF16(x), C::BF16(a), C::BF16(b)) => run!(BF16, x, a, b),
            _ => candle::bail!("unsupported dtype for rmsnorm {:?}", s1.dtype()),
        };
        Ok((out, l1.shape().clone()))
    }

    fn cuda_fwd(&self, s1: &CudaStorage, l1: &Layout, s2: &CudaStorage, l2: &Layout, s3: &CudaStorage, l3: &Layout)
        -> Result<(CudaStorage, Shape)> {
        let dt = dtype_code(s1.dtype(), "rmsnorm")?;
        if s2.dtype() != s1.dtype() || s3.dtype() != s1.dtype() {
            candle::bail!("unsupported dtype for rmsnorm {:?}", s1.dtype())
        }
        let x = base_ptr(s1, l1, "input")?;
        let alpha = base_ptr(s2, l2, "alpha")?;
        let beta = base_ptr(s3, l3, "beta")?;
        let el = l1.shape().elem_count();
        let cols = *l1.dims().last().unwrap();
        let rows = if cols == 0 { 0 } else { el / cols };
        let dev = s1.device();
        let (dst, y) = alloc_like(dev, s1.dtype(), el)?;
        check(unsafe {
            ffi::cb200_layer_norm(x, std::ptr::null(), alpha, beta, y, std::ptr::null_mut(), rows as i64, cols as i32,
                                  self.eps, dt, 0, stream(dev))
        })?;
        Ok((dst, l1.shape().clone()))
    }
}

/// `candle_nn::ops::layer_norm(xs, alpha, beta, eps)` (candle-nn/src/ops.rs:896-909).
pub fn layer_norm(xs: &Tensor, alpha: &Tensor, beta: &Tensor, eps: f32) -> Result<Tensor> {
    let hidden_size_xs = xs.dim(candle::D::Minus1)?;
    let hidden_size_alpha = alpha.dims1()?;
    let hidden_size_beta = beta.dims1()?;
    if hidden_size_xs != hidden_size_alpha || hidden_size_xs != hidden_size_beta {
        candle::bail!("shape mismatch in layer-norm src: {:?} alpha: {:?} beta: {:?}", xs.shape(), alpha.shape(), beta.shape())
    }
    xs.apply_op3_no_bwd(alpha, beta, &LayerNorm { eps })
}

// ---------------------------------------------------------------------------------------------
// The composite ("slow") norm in one launch.  On the CPU the caller keeps candle's chain of tensor ops
// (candle-nn/src/layer_norm.rs:115-135); on CUDA `LayerNorm::forward` calls this instead of that chain.
// ---------------------------------------------------------------------------------------------
#[derive(Debug, Clone)]
struct NormSlow {
    eps: f32,
    remove_mean: bool,
    has_bias: bool,
}

impl candle::CustomOp3 for NormSlow {
    fn name(&self) -> &'static str {
        "layer-norm-slow"
    }
    fn cpu_fwd(&self, _: &CpuStorage, _: &Layout, _: &CpuStorage, _: &Layout, _: &CpuStorage, _: &Layout)
        -> Result<(CpuStorage, Shape)> {
        candle::bail!("layer-norm-slow is CUDA only: on the CPU use the tensor-op chain of candle_nn::LayerNorm")
    }
    fn cuda_fwd(&self, s1: &CudaStorage, l1: &Layout, s2: &CudaStorage, l2: &Layout, s3: &CudaStorage, l3: &Layout)
        -> Result<(CudaStorage, Shape)> {
        let dt = dtype_code(s1.dtype(), "rmsnorm")?;
        let x = base_ptr(s1, l1, "input")?; // the caller made it contiguous (to_dtype does so in candle's chain)
        let w = base_ptr(s2, l2, "weight")?;
        let b = if self.has_bias { base_ptr(s3, l3, "bias")? } else { std::ptr::null() };
        let el = l1.shape().elem_count();
        let cols = *l1.dims().last().unwrap();
        let rows = if cols == 0 { 0 } else { el / cols };
        let dev = s1.device();
        let (dst, y) = alloc_like(dev, s1.dtype(), el)?;
        check(unsafe {
            ffi::cb200_layer_norm_slow(x, w, b, y, rows as i64, cols as i32, self.eps, dt, self.remove_mean as c_int, stream(dev))
        })?;
        Ok((dst, l1.shape().clone()))
    }
}

/// What `LayerNorm::forward` computes off the fused path; `bias = None` for `new_no_bias` / `rms_norm`.
pub fn norm_slow(x: &Tensor, weight: &Tensor, bias: Option<&Tensor>, eps: f64, remove_mean: bool) -> Result<Tensor> {
    let x = x.contiguous()?;
    let op = NormSlow { eps: eps as f32, remove_mean, has_bias: bias.is_some() };
    x.apply_op3_no_bwd(weight, bias.unwrap_or(weight), &op)
}
pub fn rms_norm_slow(x: &Tensor, alpha: &Tensor, eps: f32) -> Result<Tensor> {
    norm_slow(x, alpha, None, eps as f64, false)
}
pub fn layer_norm_slow(x: &Tensor, alpha: &Tensor, beta: &Tensor, eps: f32) -> Result<Tensor> {
    norm_slow(x, alpha, Some(beta), eps as f64, true)
}

// ---------------------------------------------------------------------------------------------
// softmax over the last dimension and rotary embeddings (cuda_fwd only shown; cpu_fwd stays candle's,
// candle-nn/src/ops.rs:296-333 and candle-nn/src/rotary_emb.rs:19-82, 260-327, 512-581)
// ---------------------------------------------------------------------------------------------
pub fn softmax_last_dim_cuda(s: &CudaStorage, l: &Layout) -> Result<(CudaStorage, Shape)> {
    let dt = dtype_code(s.dtype(), "softmax")?;
    let x = base_ptr(s, l, "input")?;
    let el = l.shape().elem_count();
    let cols = *l.dims().last().unwrap();
    let rows = if cols == 0 { 0 } else { el / cols };
    let dev = s.device();
    let (dst, y) = alloc_like(dev, s.dtype(), el)?;
    check(unsafe { ffi::cb200_softmax_last_dim(x, y, rows as i64, cols as i32, dt, stream(dev)) })?;
    Ok((dst, l.shape().clone()))
}

/// `variant`: ffi::ROPE_INTERLEAVED (rope_i), ROPE_HALF (rope), ROPE_THD (rope_thd); the shape and
/// contiguity checks of rotary_emb.rs:203-228 / 457-482 / 706-731 are done by the caller as today.
pub fn rope_cuda(variant: c_int, s1: &CudaStorage, l1: &Layout, s2: &CudaStorage, l2: &Layout, s3: &CudaStorage,
                 l3: &Layout) -> Result<(CudaStorage, Shape)> {
    let dt = dtype_code(s1.dtype(), "rope")?;
    let src = base_ptr(s1, l1, "input src")?;
    let cos = base_ptr(s2, l2, "input cos")?;
    let sin = base_ptr(s3, l3, "input sin")?;
    let (d0, d1, d2, d3) = l1.shape().dims4()?;
    let (b, h, t, d) = if variant == ffi::ROPE_THD { (d0, d2, d1, d3) } else { (d0, d1, d2, d3) };
    let dev = s1.device();
    let (dst, y) = alloc_like(dev, s1.dtype(), b * h * t * d)?;
    check(unsafe { ffi::cb200_rope(src, cos, sin, y, b as i64, h as i32, t as i32, d as i32, dt, variant, stream(dev)) })?;
    Ok((dst, l1.shape().clone()))
}

// ---------------------------------------------------------------------------------------------
// index_select: the body `IndexSelect::f` + `BackendStorage::index_select` get on CUDA
// (candle-core/src/cuda_backend/mod.rs:352-410, 1622-1626).  No per-call host-to-device copy of dims
// and strides; ids are bounds-checked on the device and a bad one is reported like the CPU backend's
// `Error::InvalidIndex` (cpu_backend/mod.rs:539-546) when `status` is read back.
// ---------------------------------------------------------------------------------------------
pub fn index_select_cuda(src: &CudaStorage, src_l: &Layout, ids: &CudaStorage, ids_l: &Layout, dim: usize)
    -> Result<CudaStorage> {
    let id_dtype = match ids.dtype() {
        DType::U8 => ffi::ID_U8,
        DType::U32 => ffi::ID_U32,
        DType::I64 => ffi::ID_I64,
        _ => candle::bail!("index_select ids should be u8, u32, or i64"),
    };
    let src_p = match src_l.contiguous_offsets() {
        Some(_) => base_ptr_any(src, src_l)?,
        None => Err(candle::Error::RequiresContiguous { op: "index-select" }.bt())?,
    };
    let ids_p = base_ptr(ids, ids_l, "ids")?;
    let dims = src_l.dims();
    let left: usize = dims[..dim].iter().product();
    let right: usize = dims[dim + 1..].iter().product();
    let n_ids = ids_l.shape().elem_count();
    let dev = src.device();
    let esz = src.dtype().size_in_bytes();
    let out = unsafe { dev.alloc::<u8>(left * n_ids * right * esz) }.w()?; // re-typed by the caller's Map
    let status = dev.alloc_zeros::<u8>(std::mem::size_of::<ffi::Cb200Status>()).w()?;
    check(unsafe {
        ffi::cb200_index_select(src_p, ids_p, *out.device_ptr() as *mut c_void, left as i64, dims[dim] as i64, right as i64,
                                n_ids as i64, esz as i32, id_dtype, *status.device_ptr() as *mut ffi::Cb200Status,
                                stream(dev))
    })?;
    // Deferred error: read the 32 bytes back where candle next synchronises (or here in debug builds).
    let host = dev.dtoh_sync_copy(&status).w()?;
    let st: ffi::Cb200Status = unsafe { std::ptr::read_unaligned(host.as_ptr() as *const ffi::Cb200Status) };
    if st.code == ffi::STATUS_INVALID_INDEX {
        Err(candle::Error::InvalidIndex { index: st.index as usize, size: st.size as usize, op: "index-select" }.bt())?
    }
    Ok(CudaStorage::wrap_cuda_slice(out, dev.clone()))
}

fn base_ptr_any(storage: &CudaStorage, layout: &Layout) -> Result<*const c_void> {
    base_ptr(storage, layout, "input")
}

// ---------------------------------------------------------------------------------------------
// Lookup out of a block-quantised table: a CustomOp1 on the ids tensor that carries the table, the
// trick `impl CustomOp1 for QTensor` uses for qmatmul (candle-core/src/quantized/mod.rs:464-525).
// Needs one accessor added to candle-core: `QCudaStorage::device_ptr(&self) -> u64` (its `data` field is
// private, candle-core/src/quantized/cuda.rs:9-20).
// ---------------------------------------------------------------------------------------------
pub struct QEmbedding {
    pub table: std::sync::Arc<candle::quantized::QTensor>,
    pub out_dtype: DType,
    /// `Some((alpha, eps))`: also apply rms_norm to the looked-up rows in the same launch
    pub rms_norm: Option<(Tensor, f32)>,
    /// this tensor holds rows [begin, end) of a table of `vocab` rows (0, rows, rows when unsharded)
    pub vocab_range: (usize, usize, usize),
}

impl candle::CustomOp1 for QEmbedding {
    fn name(&self) -> &'static str {
        "qembedding"
    }
    fn cpu_fwd(&self, storage: &CpuStorage, layout: &Layout) -> Result<(CpuStorage, Shape)> {
        // candle's own composition: dequantize -> to_dtype -> index_select (quantized_llama.rs:378-379,
        // embedding.rs:29-36); left to the caller on CPU devices.
        let _ = (storage, layout);
        candle::bail!("qembedding is CUDA only: on the CPU dequantize the table and use candle_nn::Embedding")
    }
    fn cuda_fwd(&self, ids: &CudaStorage, ids_l: &Layout) -> Result<(CudaStorage, Shape)> {
        let (rows, hidden) = self.table.shape().dims2()?;
        let id_dtype = match ids.dtype() {
            DType::U8 => ffi::ID_U8,
            DType::U32 => ffi::ID_U32,
            DType::I64 => ffi::ID_I64,
            _ => candle::bail!("index_select ids should be u8, u32, or i64"),
        };
        let (begin, end, vocab) = self.vocab_range;
        if end - begin != rows {
            candle::bail!("vocab shard [{begin}, {end}) does not match the table's {rows} rows")
        }
        let qtype = ggml_type_id(self.table.dtype())?;
        let qptr = qcuda_device_ptr(&self.table)? as *const c_void; // see the note above
        let ids_p = base_ptr(ids, ids_l, "ids")?;
        let n_ids = ids_l.shape().elem_count();
        let dev = ids.device();
        let dt = dtype_code(self.out_dtype, "qembedding")?;
        let (dst, y) = alloc_like(dev, self.out_dtype, n_ids * hidden)?;
        let status = dev.alloc_zeros::<u8>(std::mem::size_of::<ffi::Cb200Status>()).w()?;
        let st_p = *status.device_ptr() as *mut ffi::Cb200Status;
        match &self.rms_norm {
            None => check(unsafe {
                ffi::cb200_qembedding(qptr, qtype, ids_p, y, vocab as i64, hidden as i32, n_ids as i64, dt, id_dtype,
                                      begin as i64, end as i64, st_p, stream(dev))
            })?,
            Some((alpha, eps)) => {
                let (a_st, a_l) = alpha.storage_and_layout();
                let a_p = match &*a_st {
                    candle::Storage::Cuda(c) => base_ptr(c, a_l, "alpha")?,
                    _ => candle::bail!("alpha has to be on the same cuda device"),
                };
                check(unsafe {
                    ffi::cb200_qembedding_rms_norm(qptr, qtype, ids_p, a_p, y, std::ptr::null_mut(), vocab as i64,
                                                   hidden as i32, n_ids as i64, *eps, dt, id_dtype, begin as i64,
                                                   end as i64, 0, st_p, stream(dev))
                })?
            }
        }
        let mut dims = ids_l.shape().dims().to_vec();
        dims.push(hidden);
        Ok((dst, Shape::from(dims)))
    }
}

/// ggml type ids as in candle-core/src/quantized/mod.rs:152-171.
fn ggml_type_id(d: candle::quantized::GgmlDType) -> Result<c_int> {
    use candle::quantized::GgmlDType as G;
    Ok(match d {
        G::Q4_0 => 2, G::Q4_1 => 3, G::Q5_0 => 6, G::Q5_1 => 7, G::Q8_0 => 8,
        G::Q2K => 10, G::Q3K => 11, G::Q4K => 12, G::Q5K => 13, G::Q6K => 14, G::Q8K => 15,
        other => candle::bail!("no device decoder for {other:?}"),
    })
}

/// Placeholder for the accessor candle-core has to grow (`QTensor` -> device address of its blocks).
fn qcuda_device_ptr(_t: &candle::quantized::QTensor) -> Result<u64> {
    candle::bail!("add `pub fn device_ptr(&self) -> u64` to QCudaStorage (candle-core/src/quantized/cuda.rs) and call it here")
}

#[allow(dead_code)]
fn _uses(_: &dyn DeviceSlice<u8>) {}
