//! COMPILE-UNVERIFIED (no Rust toolchain where this was written).
//!
//! `extern "C"` declarations of include/weta_b200.h, one to one.  Only the entry points the `Backend`
//! implementation and the data-parallel trainer use are declared; the header is the authority.
#![allow(non_camel_case_types, dead_code)]

use std::os::raw::{c_char, c_int, c_void};

pub const WB_MAX_DIMS: usize = 8;

pub const WB_OK: c_int = 0;
pub const WB_ERR_DEVICE_UNAVAILABLE: c_int = 5;
pub const WB_ERR_TIMEOUT: c_int = 6;

pub const WB_F32: c_int = 0;
pub const WB_F64: c_int = 1;
pub const WB_I64: c_int = 2;

pub const WB_UNIFORM: c_int = 0;
pub const WB_NORMAL: c_int = 1;

pub const WB_MM_TF32X3: c_int = 0;
pub const WB_MM_TF32: c_int = 1;
pub const WB_MM_FP32: c_int = 2;

/// `WbView`: a strided look at device memory, offsets and strides in elements.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct WbView {
    pub data: *mut c_void,
    pub dtype: i32,
    pub ndim: i32,
    pub shape: [i64; WB_MAX_DIMS],
    pub stride: [i64; WB_MAX_DIMS],
    pub offset: i64,
}

/// `WbConvParams`: Im2ColParams flattened.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct WbConvParams {
    pub kh: i64,
    pub kw: i64,
    pub sh: i64,
    pub sw: i64,
    pub ph: i64,
    pub pw: i64,
    pub dh: i64,
    pub dw: i64,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct WbLayerSpec {
    pub kind: i32,
    pub a: i32,
    pub b: i32,
    pub c: i32,
    pub p: f64,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct WbAdamConfig {
    pub lr: f64,
    pub beta1: f64,
    pub beta2: f64,
    pub eps: f64,
    pub weight_decay: f64,
    pub decoupled: i32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct WbDpId {
    pub bytes: [u8; 128],
}

#[repr(C)]
pub struct WbBackend {
    _private: [u8; 0],
}
#[repr(C)]
pub struct WbStorage {
    _private: [u8; 0],
}
#[repr(C)]
pub struct WbTrainer {
    _private: [u8; 0],
}
#[repr(C)]
pub struct WbDp {
    _private: [u8; 0],
}

extern "C" {
    pub fn wb_device_count() -> c_int;
    pub fn wb_backend_create(ordinal: c_int, out: *mut *mut WbBackend) -> c_int;
    pub fn wb_backend_destroy(b: *mut WbBackend) -> c_int;
    pub fn wb_synchronize(b: *mut WbBackend) -> c_int;
    pub fn wb_last_error() -> *const c_char;
    pub fn wb_set_profiling(b: *mut WbBackend, on: c_int) -> c_int;
    pub fn wb_profile_report(b: *mut WbBackend) -> *const c_char;
    pub fn wb_set_matmul_mode(b: *mut WbBackend, mode: c_int) -> c_int;

    pub fn wb_alloc(b: *mut WbBackend, len: i64, dtype: c_int, out: *mut *mut WbStorage) -> c_int;
    pub fn wb_zeros(b: *mut WbBackend, len: i64, dtype: c_int, out: *mut *mut WbStorage) -> c_int;
    pub fn wb_free(b: *mut WbBackend, s: *mut WbStorage) -> c_int;
    pub fn wb_storage_data(s: *const WbStorage) -> *mut c_void;
    pub fn wb_storage_len(s: *const WbStorage) -> i64;
    pub fn wb_from_host(b: *mut WbBackend, host: *const c_void, len: i64, dtype: c_int, out: *mut *mut WbStorage) -> c_int;
    pub fn wb_to_host(b: *mut WbBackend, x: *const WbView, host_out: *mut c_void) -> c_int;

    pub fn wb_copy_strided(b: *mut WbBackend, src: *const WbView, dst: *const WbView) -> c_int;
    pub fn wb_unary(b: *mut WbBackend, op: c_int, p1: f64, p2: f64, x: *const WbView, out: *mut *mut WbStorage) -> c_int;
    pub fn wb_binary(b: *mut WbBackend, op: c_int, a: *const WbView, bb: *const WbView, out: *mut *mut WbStorage) -> c_int;
    pub fn wb_reduce(b: *mut WbBackend, op: c_int, x: *const WbView, axis: c_int, out: *mut *mut WbStorage) -> c_int;
    pub fn wb_matmul(b: *mut WbBackend, a: *const WbView, bb: *const WbView, out: *mut *mut WbStorage) -> c_int;
    pub fn wb_im2col(b: *mut WbBackend, x: *const WbView, p: *const WbConvParams, out: *mut *mut WbStorage) -> c_int;
    pub fn wb_col2im(b: *mut WbBackend, cols: *const WbView, p: *const WbConvParams, c: i64, h: i64, w: i64, out: *mut *mut WbStorage) -> c_int;
    pub fn wb_cast(b: *mut WbBackend, x: *const WbView, dtype: c_int, out: *mut *mut WbStorage) -> c_int;
    pub fn wb_random(b: *mut WbBackend, len: i64, dtype: c_int, dist: c_int, pa: f64, pb: f64, seed: u64, out: *mut *mut WbStorage) -> c_int;

    // fused training step and its data-parallel form (extension; see the header for every argument)
    pub fn wb_trainer_create(b: *mut WbBackend, layers: *const WbLayerSpec, n_layers: c_int, batch: i64, in_c: i64, in_h: i64, in_w: i64,
                             adam: *const WbAdamConfig, matmul_mode: c_int, out: *mut *mut WbTrainer) -> c_int;
    pub fn wb_trainer_destroy(t: *mut WbTrainer) -> c_int;
    pub fn wb_trainer_init(t: *mut WbTrainer, seeds: *const u64, n_seeds: c_int) -> c_int;
    pub fn wb_trainer_step_host(t: *mut WbTrainer, host_x: *const f32, host_y: *const i64, dropout_seeds: *const u64, n_seeds: c_int,
                                host_loss: *mut f32) -> c_int;
    pub fn wb_trainer_use_graph(t: *mut WbTrainer, on: c_int) -> c_int;
    pub fn wb_trainer_step(t: *mut WbTrainer, dropout_seeds: *const u64, n_seeds: c_int) -> c_int;
    pub fn wb_dp_unique_id(out: *mut WbDpId) -> c_int;
    pub fn wb_dp_create(t: *mut WbTrainer, id: *const WbDpId, rank: c_int, world: c_int, mode: c_int, bucket_elems: i64, out: *mut *mut WbDp) -> c_int;
    pub fn wb_dp_destroy(dp: *mut WbDp) -> c_int;
    pub fn wb_dp_submit(dp: *mut WbDp, pinned_x: *const f32, pinned_y: *const i64) -> c_int;
    pub fn wb_dp_step_submitted(dp: *mut WbDp, dropout_seeds: *const u64, n_seeds: c_int, host_loss: *mut f32) -> c_int;
    pub fn wb_dp_wait(dp: *mut WbDp, timeout_ms: c_int) -> c_int;
}
