//! # weta-b200
//!
//! COMPILE-UNVERIFIED: there is no Rust toolchain in the environment this file was written in.  Every
//! body is written out; expect to fix what `cargo check` finds (lifetimes, imports), not to fill gaps.
//!
//! The B200 backend: `impl Backend for B200Backend` over the C ABI of `libweta_b200.so`
//! (include/weta_b200.h), whose kernels are hand-written, AOT-compiled sm_100a code.  It has the
//! surface `weta-tensor` needs from a GPU crate and nothing else
//! (crates/weta-tensor/src/storage.rs:14, 44, 57, 68, 93, 111): `backend(ordinal)`, `B200Storage::ordinal()`,
//! `is_available()`, `device_count()`, `profile_report()`.  It mirrors crates/weta-cuda/src/lib.rs:416-680
//! method for method; where that file launches an NVRTC kernel or calls cuBLAS, this one makes one C call.
//!
//! Error behaviour follows the CUDA crate: creating a backend returns `Error::DeviceUnavailable`
//! (weta-cuda lib.rs:131-133, 176-192); every op panics on failure with the library's message, where
//! weta-cuda panics with `expect("CUDA ... failed")` (lib.rs:207, 387, 491).  There is no CPU fallback.

mod ffi;

use std::collections::HashMap;
use std::ffi::CStr;
use std::os::raw::c_void;
use std::sync::{Mutex, OnceLock};

use weta_core::{Backend, BinaryOp, DType, Device, Distribution, Error, HostData, Im2ColParams, Layout, ReduceOp, Result, UnaryOp, View};

/// Data on one B200: an arena block owned through the library's `WbStorage` handle.
pub struct B200Storage {
    handle: *mut ffi::WbStorage,
    backend: *mut ffi::WbBackend,
    dtype: DType,
    ordinal: usize,
}

// The handle is only ever used through the backend's one stream; the library's arena is mutex-protected.
unsafe impl Send for B200Storage {}
unsafe impl Sync for B200Storage {}

impl B200Storage {
    pub fn ordinal(&self) -> usize {
        self.ordinal
    }
    pub fn dtype(&self) -> DType {
        self.dtype
    }
    fn ptr(&self) -> *mut c_void {
        unsafe { ffi::wb_storage_data(self.handle) }
    }
}

impl Drop for B200Storage {
    fn drop(&mut self) {
        // The block goes back to the arena, ordered after the work already queued on the stream.
        unsafe {
            ffi::wb_free(self.backend, self.handle);
        }
    }
}

pub struct B200Backend {
    ordinal: usize,
    handle: *mut ffi::WbBackend,
}

unsafe impl Send for B200Backend {}
unsafe impl Sync for B200Backend {}

static BACKENDS: OnceLock<Mutex<HashMap<usize, &'static B200Backend>>> = OnceLock::new();

fn last_error() -> String {
    unsafe { CStr::from_ptr(ffi::wb_last_error()).to_string_lossy().into_owned() }
}

/// Panics with the library's message unless `status` is WB_OK: the counterpart of weta-cuda's `expect`s.
fn check(status: i32, what: &str) {
    if status != ffi::WB_OK {
        panic!("weta-b200: {what} failed (status {status}): {}", last_error());
    }
}

/// The backend for GPU `ordinal`, created on first use and kept for the life of the process
/// (crates/weta-cuda/src/lib.rs:137-146).  Nothing is compiled at run time.
pub fn backend(ordinal: usize) -> Result<&'static B200Backend> {
    let map = BACKENDS.get_or_init(|| Mutex::new(HashMap::new()));
    let mut map = map.lock().unwrap_or_else(|e| e.into_inner());
    if let Some(b) = map.get(&ordinal) {
        return Ok(b);
    }
    let mut handle: *mut ffi::WbBackend = std::ptr::null_mut();
    let status = unsafe { ffi::wb_backend_create(ordinal as i32, &mut handle) };
    if status != ffi::WB_OK {
        return Err(Error::DeviceUnavailable(format!("B200: {}", last_error())));
    }
    if std::env::var("WETA_CUDA_PROFILE").map(|v| v == "1").unwrap_or(false) {
        unsafe { ffi::wb_set_profiling(handle, 1) };
    }
    let b: &'static B200Backend = Box::leak(Box::new(B200Backend { ordinal, handle }));
    map.insert(ordinal, b);
    Ok(b)
}

/// The number of usable devices, or 0 if the driver can't be loaded (weta-cuda lib.rs:149-152).
pub fn device_count() -> usize {
    unsafe { ffi::wb_device_count().max(0) as usize }
}

pub fn is_available() -> bool {
    device_count() > 0
}

/// Per-op call counts and device time of every backend created so far, when profiling is on
/// (crates/weta-cuda/src/profile.rs:58-73).
pub fn profile_report() -> Option<String> {
    let map = BACKENDS.get()?;
    let map = map.lock().unwrap_or_else(|e| e.into_inner());
    let mut out = String::new();
    for (ordinal, b) in map.iter() {
        let text = unsafe { CStr::from_ptr(ffi::wb_profile_report(b.handle)).to_string_lossy().into_owned() };
        out.push_str(&format!("cuda:{ordinal}\n{text}"));
    }
    if out.is_empty() {
        None
    } else {
        Some(out)
    }
}

fn dtype_code(dt: DType) -> i32 {
    match dt {
        DType::F32 => ffi::WB_F32,
        DType::F64 => ffi::WB_F64,
        DType::I64 => ffi::WB_I64,
    }
}

/// crates/weta-cuda/src/lib.rs:256-278: the op codes the kernels switch on, with their scalar parameters.
fn unary_code(op: UnaryOp) -> (i32, f64, f64) {
    match op {
        UnaryOp::Neg => (0, 0.0, 0.0),
        UnaryOp::Exp => (1, 0.0, 0.0),
        UnaryOp::Log => (2, 0.0, 0.0),
        UnaryOp::Sqrt => (3, 0.0, 0.0),
        UnaryOp::Abs => (4, 0.0, 0.0),
        UnaryOp::Sign => (5, 0.0, 0.0),
        UnaryOp::Relu => (6, 0.0, 0.0),
        UnaryOp::Step => (7, 0.0, 0.0),
        UnaryOp::Tanh => (8, 0.0, 0.0),
        UnaryOp::Sigmoid => (9, 0.0, 0.0),
        UnaryOp::Erf => (10, 0.0, 0.0),
        UnaryOp::Sin => (11, 0.0, 0.0),
        UnaryOp::Cos => (12, 0.0, 0.0),
        UnaryOp::Recip => (13, 0.0, 0.0),
        UnaryOp::Affine { mul, add } => (14, mul, add),
        UnaryOp::Powf(e) => (15, e, 0.0),
        UnaryOp::GtScalar(v) => (16, v, 0.0),
        UnaryOp::MaxScalar(v) => (17, v, 0.0),
        UnaryOp::MinScalar(v) => (18, v, 0.0),
    }
}

/// crates/weta-cuda/src/lib.rs:280-296
fn binary_code(op: BinaryOp) -> i32 {
    match op {
        BinaryOp::Add => 0,
        BinaryOp::Sub => 1,
        BinaryOp::Mul => 2,
        BinaryOp::Div => 3,
        BinaryOp::Pow => 4,
        BinaryOp::Maximum => 5,
        BinaryOp::Minimum => 6,
        BinaryOp::Eq => 7,
        BinaryOp::Ne => 8,
        BinaryOp::Lt => 9,
        BinaryOp::Le => 10,
        BinaryOp::Gt => 11,
        BinaryOp::Ge => 12,
    }
}

fn reduce_code(op: ReduceOp) -> i32 {
    match op {
        ReduceOp::Sum => 0,
        ReduceOp::Max => 1,
        ReduceOp::Min => 2,
        ReduceOp::ArgMax => 3,
        ReduceOp::ArgMin => 4,
    }
}

/// A `WbView` of `storage` through `layout` (the counterpart of `Strides::of`, weta-cuda lib.rs:65-79).
fn view_of(ptr: *mut c_void, layout: &Layout, dtype: DType) -> ffi::WbView {
    assert!(layout.ndim() <= ffi::WB_MAX_DIMS, "the B200 backend supports at most 8 dims, got shape {:?}", layout.shape());
    let mut v = ffi::WbView { data: ptr, dtype: dtype_code(dtype), ndim: layout.ndim() as i32, shape: [1; 8], stride: [0; 8], offset: layout.offset() as i64 };
    for i in 0..layout.ndim() {
        v.shape[i] = layout.shape()[i] as i64;
        v.stride[i] = layout.strides()[i] as i64;
    }
    v
}

fn view(x: &View<'_, B200Storage>) -> ffi::WbView {
    view_of(x.storage.ptr(), x.layout, x.dtype)
}

fn conv_params(p: Im2ColParams) -> ffi::WbConvParams {
    let i = |v: usize| v as i64;
    ffi::WbConvParams { kh: i(p.kernel.0), kw: i(p.kernel.1), sh: i(p.stride.0), sw: i(p.stride.1), ph: i(p.padding.0), pw: i(p.padding.1),
                        dh: i(p.dilation.0), dw: i(p.dilation.1) }
}

impl B200Backend {
    fn wrap(&self, handle: *mut ffi::WbStorage, dtype: DType) -> B200Storage {
        B200Storage { handle, backend: self.handle, dtype, ordinal: self.ordinal }
    }

    /// Contractions: TF32 tensor cores with three products per term (FP32-grade, the default), one product per
    /// term, or FP32 CUDA cores.  The reference calls cuBLAS in its default FP32 mode (weta-cuda lib.rs:351-389).
    pub fn set_matmul_mode(&self, mode: i32) {
        check(unsafe { ffi::wb_set_matmul_mode(self.handle, mode) }, "set_matmul_mode");
    }

    pub fn synchronize(&self) {
        check(unsafe { ffi::wb_synchronize(self.handle) }, "synchronize");
    }

    /// The raw handle, for the fused-trainer and data-parallel entry points (`wb_trainer_*`, `wb_dp_*`).
    pub fn raw(&self) -> *mut c_void {
        self.handle as *mut c_void
    }
}

impl Backend for B200Backend {
    type Storage = B200Storage;

    fn device(&self) -> Device {
        Device::Cuda(self.ordinal)
    }

    fn from_host(&self, data: HostData) -> B200Storage {
        let mut out: *mut ffi::WbStorage = std::ptr::null_mut();
        let (ptr, len, dt) = match &data {
            HostData::F32(v) => (v.as_ptr() as *const c_void, v.len(), DType::F32),
            HostData::F64(v) => (v.as_ptr() as *const c_void, v.len(), DType::F64),
            HostData::I64(v) => (v.as_ptr() as *const c_void, v.len(), DType::I64),
        };
        // Pageable memory is staged before the call returns, so `data` may be dropped right after.
        check(unsafe { ffi::wb_from_host(self.handle, ptr, len as i64, dtype_code(dt), &mut out) }, "from_host");
        self.wrap(out, dt)
    }

    fn to_host(&self, x: View<'_, B200Storage>) -> HostData {
        let n = x.layout.numel();
        let v = view(&x);
        match x.dtype {
            DType::F32 => {
                let mut host = vec![0f32; n];
                check(unsafe { ffi::wb_to_host(self.handle, &v, host.as_mut_ptr() as *mut c_void) }, "to_host");
                HostData::F32(host)
            }
            DType::F64 => {
                let mut host = vec![0f64; n];
                check(unsafe { ffi::wb_to_host(self.handle, &v, host.as_mut_ptr() as *mut c_void) }, "to_host");
                HostData::F64(host)
            }
            DType::I64 => {
                let mut host = vec![0i64; n];
                check(unsafe { ffi::wb_to_host(self.handle, &v, host.as_mut_ptr() as *mut c_void) }, "to_host");
                HostData::I64(host)
            }
        }
    }

    fn zeros(&self, len: usize, dtype: DType) -> B200Storage {
        let mut out: *mut ffi::WbStorage = std::ptr::null_mut();
        check(unsafe { ffi::wb_zeros(self.handle, len as i64, dtype_code(dtype), &mut out) }, "zeros");
        self.wrap(out, dtype)
    }

    fn copy_strided(&self, src: View<'_, B200Storage>, dst: &mut B200Storage, dst_layout: &Layout) {
        if src.layout.numel() == 0 {
            return;
        }
        assert!(src.dtype == dst.dtype, "copy: dtype mismatch");
        let (s, d) = (view(&src), view_of(dst.ptr(), dst_layout, dst.dtype));
        check(unsafe { ffi::wb_copy_strided(self.handle, &s, &d) }, "copy_strided");
    }

    fn unary(&self, op: UnaryOp, x: View<'_, B200Storage>) -> B200Storage {
        let (code, p1, p2) = unary_code(op);
        let mut out: *mut ffi::WbStorage = std::ptr::null_mut();
        let v = view(&x);
        // i64 tensors accept only the ops weta-cpu defines for them (crates/weta-cpu/src/lib.rs:190-203); the library
        // returns WB_ERR_UNSUPPORTED for the rest, which panics here like the CPU backend does.
        check(unsafe { ffi::wb_unary(self.handle, code, p1, p2, &v, &mut out) }, "unary");
        self.wrap(out, x.dtype)
    }

    fn binary(&self, op: BinaryOp, a: View<'_, B200Storage>, b: View<'_, B200Storage>) -> B200Storage {
        assert!(a.dtype == b.dtype, "binary: dtype mismatch");
        let mut out: *mut ffi::WbStorage = std::ptr::null_mut();
        let (va, vb) = (view(&a), view(&b));
        check(unsafe { ffi::wb_binary(self.handle, binary_code(op), &va, &vb, &mut out) }, "binary");
        self.wrap(out, a.dtype)
    }

    fn reduce(&self, op: ReduceOp, x: View<'_, B200Storage>, axis: usize) -> B200Storage {
        let mut out: *mut ffi::WbStorage = std::ptr::null_mut();
        let v = view(&x);
        check(unsafe { ffi::wb_reduce(self.handle, reduce_code(op), &v, axis as i32, &mut out) }, "reduce");
        let dt = match op {
            ReduceOp::ArgMax | ReduceOp::ArgMin => DType::I64,
            _ => x.dtype,
        };
        self.wrap(out, dt)
    }

    fn matmul(&self, a: View<'_, B200Storage>, b: View<'_, B200Storage>) -> B200Storage {
        assert!(a.dtype == b.dtype, "matmul: dtype mismatch");
        let mut out: *mut ffi::WbStorage = std::ptr::null_mut();
        let (va, vb) = (view(&a), view(&b));
        // Any strides, batch stride 0 included: no operand is copied or transposed in memory.
        check(unsafe { ffi::wb_matmul(self.handle, &va, &vb, &mut out) }, "matmul");
        self.wrap(out, a.dtype)
    }

    fn im2col(&self, x: View<'_, B200Storage>, p: Im2ColParams) -> B200Storage {
        let mut out: *mut ffi::WbStorage = std::ptr::null_mut();
        let (v, cp) = (view(&x), conv_params(p));
        check(unsafe { ffi::wb_im2col(self.handle, &v, &cp, &mut out) }, "im2col");
        self.wrap(out, x.dtype)
    }

    fn col2im(&self, cols: View<'_, B200Storage>, p: Im2ColParams, chw: (usize, usize, usize)) -> B200Storage {
        let mut out: *mut ffi::WbStorage = std::ptr::null_mut();
        let (v, cp) = (view(&cols), conv_params(p));
        check(unsafe { ffi::wb_col2im(self.handle, &v, &cp, chw.0 as i64, chw.1 as i64, chw.2 as i64, &mut out) }, "col2im");
        self.wrap(out, cols.dtype)
    }

    fn cast(&self, x: View<'_, B200Storage>, dtype: DType) -> B200Storage {
        let mut out: *mut ffi::WbStorage = std::ptr::null_mut();
        let v = view(&x);
        check(unsafe { ffi::wb_cast(self.handle, &v, dtype_code(dtype), &mut out) }, "cast");
        self.wrap(out, dtype)
    }

    /// Filled on the device: uniform fills are bit-identical to the CPU backend, normal fills wherever the CPU's
    /// libm rounds `ln` and `cos` correctly (crates/weta-core/src/ops.rs:176-189).
    fn random(&self, len: usize, dtype: DType, dist: Distribution, seed: u64) -> B200Storage {
        if dtype == DType::I64 {
            panic!("random: expected a float dtype, got i64");
        }
        let (kind, a, b) = match dist {
            Distribution::Uniform { lo, hi } => (ffi::WB_UNIFORM, lo, hi),
            Distribution::Normal { mean, std } => (ffi::WB_NORMAL, mean, std),
        };
        let mut out: *mut ffi::WbStorage = std::ptr::null_mut();
        check(unsafe { ffi::wb_random(self.handle, len as i64, dtype_code(dtype), kind, a, b, seed, &mut out) }, "random");
        self.wrap(out, dtype)
    }
}
