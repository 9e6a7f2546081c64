//! candle-shaped `QTensor` / `QMatMul` over `libturq.so`.
//!
//! tur reaches its quantized linears through three candle items
//! (`src/models/layers/linear.rs:1-32,62-69`, `src/weights/gguf_varbuilder.rs:52-94`):
//! `QMatMul::from_arc(Arc<QTensor>)`, `Module::forward(&self, &Tensor)` and
//! `QTensor::{dequantize, shape}`. This crate keeps those names and their error behaviour
//! (`Result` everywhere, no `unwrap` / `expect` / `panic`: the reference denies them,
//! `Cargo.toml:79-86`, and builds with `panic = "abort"`, `Cargo.toml:175`) on top of the
//! flat C ABI of `turq-sys`. Activations are host slices here, as they are in tur today
//! (`Device::Cpu` everywhere: `tests/common.rs:5`); the `*_device` methods take raw device
//! pointers for a host that already keeps its tensors on the GPU.
//!
//! This file has not been compiled in the image it was written in (no Rust toolchain
//! there); the same ABI is exercised end to end by the Python ctypes layer and the C++
//! header `include/turq.hpp`.

use core::ffi::{c_char, c_void};
use std::ffi::CStr;
use std::fmt;
use std::ptr;
use std::sync::Arc;

use turq_sys as sys;

/// A non-zero `turq_status` with the library's message for it.
#[derive(Debug, Clone)]
pub struct Error {
    pub status: i32,
    pub message: String,
}

impl fmt::Display for Error {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        write!(f, "turq status {}: {}", self.status, self.message)
    }
}

impl std::error::Error for Error {}

pub type Result<T> = core::result::Result<T, Error>;

fn c_str(p: *const c_char) -> String {
    if p.is_null() {
        return String::new();
    }
    // SAFETY: the library returns NUL-terminated strings that live as long as the context
    // (turq_last_error) or the library image (turq_status_string).
    unsafe { CStr::from_ptr(p) }.to_string_lossy().into_owned()
}

/// GGUF tensor type ids (candle: `GgmlDType`).
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
#[repr(i32)]
pub enum GgmlDType {
    F32 = sys::TURQ_F32,
    F16 = sys::TURQ_F16,
    Q8_0 = sys::TURQ_Q8_0,
    Q4K = sys::TURQ_Q4_K,
    Q5K = sys::TURQ_Q5_K,
    Q6K = sys::TURQ_Q6_K,
    Q8K = sys::TURQ_Q8_K,
    BF16 = sys::TURQ_BF16,
}

impl GgmlDType {
    pub fn from_u32(v: u32) -> Result<Self> {
        Ok(match v as i32 {
            sys::TURQ_F32 => Self::F32,
            sys::TURQ_F16 => Self::F16,
            sys::TURQ_Q8_0 => Self::Q8_0,
            sys::TURQ_Q4_K => Self::Q4K,
            sys::TURQ_Q5_K => Self::Q5K,
            sys::TURQ_Q6_K => Self::Q6K,
            sys::TURQ_Q8_K => Self::Q8K,
            sys::TURQ_BF16 => Self::BF16,
            _ => {
                return Err(Error { status: sys::TURQ_E_DTYPE, message: format!("unknown GGUF dtype {v}") });
            }
        })
    }

    /// Elements per block (candle: `GgmlDType::block_size`).
    pub fn block_size(self) -> usize {
        // SAFETY: pure function of its argument.
        unsafe { sys::turq_block_elems(self as i32) as usize }
    }

    /// Bytes per block (candle: `GgmlDType::type_size`).
    pub fn type_size(self) -> usize {
        // SAFETY: pure function of its argument.
        unsafe { sys::turq_block_bytes(self as i32) as usize }
    }
}

/// How `QMatMul::forward` computes (see `turq_mode` in turq.h).
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
#[repr(i32)]
pub enum Mode {
    Auto = sys::TURQ_MODE_AUTO,
    Int8Act = sys::TURQ_MODE_INT8_ACT,
    ExactF32 = sys::TURQ_MODE_EXACT_F32,
    TensorCore = sys::TURQ_MODE_TENSOR_CORE,
}

/// One CUDA device with the scratch memory of the calls made through it. tur runs one
/// worker thread per model (`src/server/worker.rs:63-72`): give each its own context.
pub struct Context {
    h: *mut sys::turq_ctx,
}

// SAFETY: the handle may move between threads; calls through one context are serialised by
// `&self` users holding it behind their own synchronisation, as the C ABI requires (one
// thread and one stream at a time per context).
unsafe impl Send for Context {}
unsafe impl Sync for Context {}

impl Context {
    pub fn new(device: i32) -> Result<Arc<Self>> {
        let mut h: *mut sys::turq_ctx = ptr::null_mut();
        // SAFETY: `h` is a valid out pointer.
        let st = unsafe { sys::turq_ctx_create(device, &mut h) };
        if st != sys::TURQ_OK || h.is_null() {
            // SAFETY: pure function of its argument.
            let msg = c_str(unsafe { sys::turq_status_string(st) });
            return Err(Error { status: st, message: format!("turq_ctx_create(device = {device}): {msg}") });
        }
        Ok(Arc::new(Self { h }))
    }

    fn check(&self, st: i32) -> Result<()> {
        if st == sys::TURQ_OK {
            return Ok(());
        }
        // SAFETY: `self.h` is a live context.
        let message = c_str(unsafe { sys::turq_last_error(self.h) });
        Err(Error { status: st, message })
    }

    /// Sizes the scratch for the largest call, so that no later call allocates.
    pub fn reserve(&self, max_m: usize, max_k: usize, max_n: usize) -> Result<()> {
        // SAFETY: live context, plain integers.
        self.check(unsafe { sys::turq_ctx_reserve(self.h, max_m as i64, max_k as i64, max_n as i64) })
    }

    /// Pins what `Mode::Auto` means to one scheme for every row count (tur expects a token's
    /// result not to depend on its batch or chunk: `tests/pipeline_integration.rs:275-369`).
    pub fn set_auto_policy(&self, mode: Mode) -> Result<()> {
        // SAFETY: live context.
        self.check(unsafe { sys::turq_ctx_set_auto_policy(self.h, mode as i32) })
    }

    /// Synchronizes `stream` and reports a kernel that gave up a bounded device-side wait.
    pub fn poll_status(&self, stream: *mut c_void) -> Result<()> {
        // SAFETY: live context; `stream` is a cudaStream_t or null.
        self.check(unsafe { sys::turq_ctx_poll_status(self.h, stream) })
    }
}

impl Drop for Context {
    fn drop(&mut self) {
        // SAFETY: the handle was created by turq_ctx_create and is dropped once.
        unsafe {
            sys::turq_ctx_destroy(self.h);
        }
    }
}

/// An immutable quantized weight `[rows, cols]` resident on one GPU (candle: `QTensor`).
pub struct QTensor {
    h: *mut sys::turq_qtensor,
    ctx: Arc<Context>,
    dtype: GgmlDType,
    shape: (usize, usize),
    nbytes: usize,
}

// SAFETY: immutable after upload; the library never writes through the handle again.
unsafe impl Send for QTensor {}
unsafe impl Sync for QTensor {}

impl QTensor {
    /// From GGUF wire-format blocks in host memory (what `gguf_file::Content::tensor` reads,
    /// `src/weights/gguf_varbuilder.rs:73`).
    pub fn new(ctx: &Arc<Context>, blocks: &[u8], dtype: GgmlDType, shape: (usize, usize)) -> Result<Self> {
        let mut h: *mut sys::turq_qtensor = ptr::null_mut();
        // SAFETY: `blocks` outlives the call (the upload is synchronous), `h` is a valid out pointer.
        let st = unsafe {
            sys::turq_qtensor_from_host(
                ctx.h,
                dtype as i32,
                shape.0 as i64,
                shape.1 as i64,
                blocks.as_ptr().cast::<c_void>(),
                blocks.len(),
                &mut h,
            )
        };
        ctx.check(st)?;
        Self::wrap(ctx, h)
    }

    /// candle: `QTensor::quantize(&Tensor, GgmlDType)`. `src` holds `shape.0` rows of `shape.1` f32
    /// values; the blocks are computed on the device (`turq_quantize_weights`) and converted to
    /// the device layout without returning to the host.
    pub fn quantize(ctx: &Arc<Context>, src: &[f32], dtype: GgmlDType, shape: (usize, usize)) -> Result<Self> {
        let n = shape.0.checked_mul(shape.1).ok_or(Error { status: sys::TURQ_E_SHAPE, message: "shape overflows".into() })?;
        if src.len() != n || n == 0 {
            return Err(Error { status: sys::TURQ_E_SHAPE, message: format!("{} values for shape {:?}", src.len(), shape) });
        }
        // SAFETY: pure size query.
        let nbytes = unsafe { sys::turq_row_bytes(dtype as i32, shape.1 as i64) } * shape.0;
        if nbytes == 0 {
            return Err(Error { status: sys::TURQ_E_SHAPE, message: format!("{} columns are not whole blocks", shape.1) });
        }
        let (mut dev_x, mut dev_b): (*mut c_void, *mut c_void) = (ptr::null_mut(), ptr::null_mut());
        let mut h: *mut sys::turq_qtensor = ptr::null_mut();
        // SAFETY: plain allocation / copy calls of the CUDA runtime and library calls on live
        // handles; both device buffers are released on every path. The null stream orders the
        // copy, the two library launches and the synchronous free.
        let st = unsafe {
            if cuda::cudaMalloc(&mut dev_x, n * 4) != 0 {
                return Err(Error { status: sys::TURQ_E_CUDA, message: "cudaMalloc failed".into() });
            }
            if cuda::cudaMalloc(&mut dev_b, nbytes) != 0 {
                cuda::cudaFree(dev_x);
                return Err(Error { status: sys::TURQ_E_CUDA, message: "cudaMalloc failed".into() });
            }
            let mut st = if cuda::cudaMemcpy(dev_x, src.as_ptr().cast::<c_void>(), n * 4, cuda::MEMCPY_HOST_TO_DEVICE) == 0 {
                sys::turq_quantize_weights(ctx.h, dtype as i32, dev_x.cast::<f32>(), shape.0 as i64, shape.1 as i64, dev_b, ptr::null_mut())
            } else {
                sys::TURQ_E_CUDA
            };
            if st == sys::TURQ_OK {
                st = sys::turq_qtensor_from_device(ctx.h, dtype as i32, shape.0 as i64, shape.1 as i64, dev_b, nbytes, ptr::null_mut(), &mut h);
            }
            cuda::cudaFree(dev_x);
            cuda::cudaFree(dev_b);
            st
        };
        ctx.check(st)?;
        Self::wrap(ctx, h)
    }

    fn wrap(ctx: &Arc<Context>, h: *mut sys::turq_qtensor) -> Result<Self> {
        let (mut dt, mut r, mut c, mut nb) = (0i32, 0i64, 0i64, 0usize);
        // SAFETY: `h` is a live tensor handle, the out pointers are valid.
        let st = unsafe { sys::turq_qtensor_info(h, &mut dt, &mut r, &mut c, &mut nb) };
        if st != sys::TURQ_OK {
            // SAFETY: `h` came from the library and is released exactly once.
            unsafe {
                sys::turq_qtensor_free(h);
            }
            return Err(match ctx.check(st) {
                Err(e) => e,
                Ok(()) => Error { status: st, message: String::new() },
            });
        }
        Ok(Self { h, ctx: Arc::clone(ctx), dtype: GgmlDType::from_u32(dt as u32)?, shape: (r as usize, c as usize), nbytes: nb })
    }

    pub fn dtype(&self) -> GgmlDType {
        self.dtype
    }

    /// `(out_features, in_features)` (candle: `QTensor::shape`, checked at `gguf_varbuilder.rs:78-84`).
    pub fn shape(&self) -> (usize, usize) {
        self.shape
    }

    pub fn storage_size_in_bytes(&self) -> usize {
        self.nbytes
    }

    /// `QTensor::dequantize` (`src/weights/mod.rs:150,161`): the f32 values, row-major, on the host.
    pub fn dequantize(&self) -> Result<Vec<f32>> {
        let n = self.shape.0 * self.shape.1;
        let mut out = vec![0f32; n];
        // the library writes into device memory; this method owns that buffer for the call
        let mut dev: *mut c_void = ptr::null_mut();
        // SAFETY: plain allocation / copy calls of the CUDA runtime, checked below.
        unsafe {
            if cuda::cudaMalloc(&mut dev, n * 4) != 0 {
                return Err(Error { status: sys::TURQ_E_CUDA, message: "cudaMalloc failed".into() });
            }
            let st = sys::turq_dequantize(self.ctx.h, self.h, sys::TURQ_F32, dev, ptr::null_mut());
            let copied = cuda::cudaMemcpy(out.as_mut_ptr().cast::<c_void>(), dev, n * 4, cuda::MEMCPY_DEVICE_TO_HOST);
            cuda::cudaFree(dev);
            self.ctx.check(st)?;
            if copied != 0 {
                return Err(Error { status: sys::TURQ_E_CUDA, message: "cudaMemcpy failed".into() });
            }
        }
        Ok(out)
    }

    /// Rows `[row0, row0 + n)` as a tensor of their own (column-parallel shard).
    pub fn slice_rows(&self, row0: usize, n: usize) -> Result<Self> {
        let mut h: *mut sys::turq_qtensor = ptr::null_mut();
        // SAFETY: live handles, valid out pointer.
        let st = unsafe { sys::turq_qtensor_slice_rows(self.ctx.h, self.h, row0 as i64, n as i64, &mut h) };
        self.ctx.check(st)?;
        Self::wrap(&self.ctx, h)
    }

    /// Columns `[col0, col0 + n)` in whole blocks (row-parallel shard).
    pub fn slice_cols(&self, col0: usize, n: usize) -> Result<Self> {
        let mut h: *mut sys::turq_qtensor = ptr::null_mut();
        // SAFETY: live handles, valid out pointer.
        let st = unsafe { sys::turq_qtensor_slice_cols(self.ctx.h, self.h, col0 as i64, n as i64, &mut h) };
        self.ctx.check(st)?;
        Self::wrap(&self.ctx, h)
    }
}

impl Drop for QTensor {
    fn drop(&mut self) {
        if !self.h.is_null() {
            // SAFETY: the handle came from the library and is released exactly once.
            unsafe {
                sys::turq_qtensor_free(self.h);
            }
        }
    }
}

/// The three CUDA runtime calls `QTensor::quantize` / `dequantize` need to move host values.
mod cuda {
    use core::ffi::c_void;
    pub const MEMCPY_HOST_TO_DEVICE: i32 = 1;
    pub const MEMCPY_DEVICE_TO_HOST: i32 = 2;
    #[link(name = "cudart")]
    unsafe extern "C" {
        pub fn cudaMalloc(ptr: *mut *mut c_void, bytes: usize) -> i32;
        pub fn cudaFree(ptr: *mut c_void) -> i32;
        pub fn cudaMemcpy(dst: *mut c_void, src: *const c_void, bytes: usize, kind: i32) -> i32;
    }
}

/// `y = x . W^T` for a quantized `W` (candle: `QMatMul`). `Clone` is a reference-count bump, as
/// `LinearX: Clone` needs (`src/models/layers/linear.rs:8`).
#[derive(Clone)]
pub struct QMatMul {
    w: Arc<QTensor>,
    mode: Mode,
}

impl QMatMul {
    /// `QMatMul::from_arc` (`src/models/layers/linear.rs:69`).
    pub fn from_arc(w: Arc<QTensor>) -> Result<Self> {
        Ok(Self { w, mode: Mode::Auto })
    }

    pub fn from_qtensor(w: QTensor) -> Result<Self> {
        Self::from_arc(Arc::new(w))
    }

    pub fn with_mode(mut self, mode: Mode) -> Self {
        self.mode = mode;
        self
    }

    /// `Module::forward` (`linear.rs:24`) plus the bias add of `LinearX::forward`
    /// (`linear.rs:25-28`): `x` is `[m, in_features]` row-major on the host, the result
    /// `[m, out_features]`.
    pub fn forward(&self, x: &[f32], bias: Option<&[f32]>) -> Result<Vec<f32>> {
        let (n, k) = self.w.shape;
        if k == 0 || x.len() % k != 0 || x.is_empty() {
            return Err(Error {
                status: sys::TURQ_E_SHAPE,
                message: format!("x has {} elements, not a positive multiple of in-features {k}", x.len()),
            });
        }
        if let Some(b) = bias {
            if b.len() != n {
                return Err(Error { status: sys::TURQ_E_SHAPE, message: format!("bias has {} elements, expected {n}", b.len()) });
            }
        }
        let m = x.len() / k;
        let mut y = vec![0f32; m * n];
        // SAFETY: x, y and bias are live for the duration of the (synchronous) call and sized as the
        // library expects: [m, k], [m, n], [n].
        let st = unsafe {
            sys::turq_qmatmul_host(
                self.w.ctx.h,
                self.w.h,
                x.as_ptr(),
                m as i64,
                y.as_mut_ptr(),
                self.mode as i32,
                bias.map_or(ptr::null(), <[f32]>::as_ptr),
            )
        };
        self.w.ctx.check(st)?;
        Ok(y)
    }

    /// Several linears that read the same `x` (attn_q|k|v: `src/models/qwen3.rs:272-274`;
    /// ffn_gate|up: `qwen3.rs:162-166`) in one round trip.
    pub fn forward_multi(mms: &[&QMatMul], x: &[f32]) -> Result<Vec<Vec<f32>>> {
        let first = mms.first().ok_or_else(|| Error { status: sys::TURQ_E_INVALID_ARG, message: "no weights".into() })?;
        let k = first.w.shape.1;
        if mms.len() > 4 || k == 0 || x.is_empty() || x.len() % k != 0 {
            return Err(Error { status: sys::TURQ_E_SHAPE, message: "1..4 weights and x of m * in-features elements".into() });
        }
        let m = x.len() / k;
        let mut ys: Vec<Vec<f32>> = mms.iter().map(|mm| vec![0f32; m * mm.w.shape.0]).collect();
        let qts: Vec<*const sys::turq_qtensor> = mms.iter().map(|mm| mm.w.h.cast_const()).collect();
        let yps: Vec<*mut f32> = ys.iter_mut().map(|y| y.as_mut_ptr()).collect();
        // SAFETY: pointer arrays and buffers are live and sized [count], [m, k], [m, n_i].
        let st = unsafe {
            sys::turq_qmatmul_multi_host(
                first.w.ctx.h,
                mms.len() as i32,
                qts.as_ptr(),
                x.as_ptr(),
                m as i64,
                yps.as_ptr(),
                first.mode as i32,
                ptr::null(),
            )
        };
        first.w.ctx.check(st)?;
        Ok(ys)
    }

    /// The same product on device memory: `dev_x` is `[m, in_features]` f32 on the weight's
    /// device, `dev_y` `[m, out_features]` f32, `stream` a `cudaStream_t` (null = default).
    ///
    /// # Safety
    /// The pointers must be device pointers on the weight's device with the stated sizes, and
    /// stay valid until the stream has run the work.
    pub unsafe fn forward_device(&self, dev_x: *const f32, m: usize, dev_y: *mut f32, dev_bias: *const f32, stream: *mut c_void) -> Result<()> {
        // SAFETY: forwarded contract of this function.
        let st = unsafe {
            sys::turq_qmatmul(self.w.ctx.h, self.w.h, dev_x.cast::<c_void>(), sys::TURQ_F32, m as i64, dev_y, self.mode as i32, dev_bias, stream)
        };
        self.w.ctx.check(st)
    }
}

/// tur's quantized linear (`LinearX::Quantized { qmatmul, bias }`, `linear.rs:13-16`).
#[derive(Clone)]
pub struct LinearX {
    pub qmatmul: QMatMul,
    pub bias: Option<Arc<Vec<f32>>>,
}

impl LinearX {
    pub fn forward(&self, x: &[f32]) -> Result<Vec<f32>> {
        self.qmatmul.forward(x, self.bias.as_deref().map(Vec::as_slice))
    }
}
