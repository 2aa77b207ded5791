//! NOT COMPILED IN THIS ENVIRONMENT (no Rust toolchain here).
//!
//! `extern "C"` declarations for every symbol of `include/oxmera_b200.h`, in
//! the header's order.  A test of the CUDA repository checks that the names
//! declared here are exactly the header's.

#![allow(non_camel_case_types)]

use std::os::raw::{c_char, c_double, c_float, c_int, c_void};

pub const OXM_MAX_DIMS: usize = 8;

// oxm_dtype: 0..5 are oxmera's DType in declaration order (dtype.rs:9-22).
pub const OXM_F32: i32 = 0;
pub const OXM_F64: i32 = 1;
pub const OXM_I32: i32 = 2;
pub const OXM_I64: i32 = 3;
pub const OXM_U8: i32 = 4;
pub const OXM_BOOL: i32 = 5;
pub const OXM_BF16: i32 = 6;
pub const OXM_F16: i32 = 7;
pub const OXM_F8E4M3: i32 = 8;
pub const OXM_F8E5M2: i32 = 9;

// oxm_status: 1..9 are the variants of oxmera_core::Error in declaration order (error.rs:12-102).
pub const OXM_OK: c_int = 0;
pub const OXM_SHAPE_MISMATCH: c_int = 1;
pub const OXM_BROADCAST_INCOMPATIBLE: c_int = 2;
pub const OXM_DTYPE_MISMATCH: c_int = 3;
pub const OXM_UNSUPPORTED_DTYPE: c_int = 4;
pub const OXM_DEVICE_MISMATCH: c_int = 5;
pub const OXM_INDEX_OUT_OF_BOUNDS: c_int = 6;
pub const OXM_RANK_MISMATCH: c_int = 7;
pub const OXM_BACKEND_UNAVAILABLE: c_int = 8;
pub const OXM_NOT_IMPLEMENTED: c_int = 9;
pub const OXM_CUDA_ERROR: c_int = 10;
pub const OXM_TIMEOUT: c_int = 11;
pub const OXM_INVALID_ARGUMENT: c_int = 12;
pub const OXM_DIVIDE_BY_ZERO: c_int = 13;

pub const OXM_ACT_NONE: i32 = 0;
pub const OXM_ACT_RELU: i32 = 1;
pub const OXM_ACT_GELU: i32 = 2;

pub const OXM_NEG: c_int = 0;
pub const OXM_EXP: c_int = 1;
pub const OXM_LN: c_int = 2;
pub const OXM_ABS: c_int = 3;
pub const OXM_ADD: c_int = 0;
pub const OXM_SUB: c_int = 1;
pub const OXM_MUL: c_int = 2;
pub const OXM_DIV: c_int = 3;
pub const OXM_SUM: c_int = 0;
pub const OXM_MAX: c_int = 1;

pub const OXM_NOALLOC_SCRATCH_BYTES: usize = 32 << 20;

/// `oxm_view`: oxmera's `Layout {shape, strides, offset}` (layout.rs:26-34; signed
/// element strides, offset in elements) plus the device pointer and device
/// index of the `Storage` behind it.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct oxm_view {
    pub dtype: i32,
    pub ndim: i32,
    pub shape: [i64; OXM_MAX_DIMS],
    pub strides: [i64; OXM_MAX_DIMS],
    pub offset: i64,
    pub base: *mut c_void,
    pub device: i32,
    pub reserved: i32,
}

/// `oxm_epilogue`
#[repr(C)]
pub struct oxm_epilogue {
    pub bias: *const oxm_view,
    pub activation: i32,
    pub accumulate: i32,
}

#[repr(C)]
pub struct oxm_ctx {
    _private: [u8; 0],
}
#[repr(C)]
pub struct oxm_event {
    _private: [u8; 0],
}

extern "C" {
    // ---- backend identity and lifetime ----
    pub fn oxm_device_count(count: *mut c_int) -> c_int;
    pub fn oxm_ctx_create(device_index: c_int, out: *mut *mut oxm_ctx) -> c_int;
    pub fn oxm_ctx_destroy(ctx: *mut oxm_ctx) -> c_int;
    pub fn oxm_ctx_device(ctx: *const oxm_ctx, device_index: *mut c_int) -> c_int;
    pub fn oxm_backend_name() -> *const c_char;
    pub fn oxm_last_error() -> *const c_char;
    pub fn oxm_status_name(status: c_int) -> *const c_char;

    // ---- storage ----
    pub fn oxm_alloc(ctx: *mut oxm_ctx, bytes: usize, out: *mut *mut c_void) -> c_int;
    pub fn oxm_free(ctx: *mut oxm_ctx, ptr: *mut c_void) -> c_int;
    pub fn oxm_h2d(ctx: *mut oxm_ctx, dst_device: *mut c_void, src_host: *const c_void, bytes: usize) -> c_int;
    pub fn oxm_d2h(ctx: *mut oxm_ctx, dst_host: *mut c_void, src_device: *const c_void, bytes: usize) -> c_int;
    pub fn oxm_memset(ctx: *mut oxm_ctx, dst_device: *mut c_void, byte: c_int, bytes: usize) -> c_int;
    pub fn oxm_copy_peer(dst_ctx: *mut oxm_ctx, dst_device: *mut c_void, src_ctx: *mut oxm_ctx, src_device: *const c_void, bytes: usize) -> c_int;
    pub fn oxm_sync(ctx: *mut oxm_ctx) -> c_int;
    pub fn oxm_host_alloc(bytes: usize, out: *mut *mut c_void) -> c_int;
    pub fn oxm_host_free(ptr: *mut c_void) -> c_int;

    // ---- the operator surface ----
    pub fn oxm_matmul(ctx: *mut oxm_ctx, a: *const oxm_view, b: *const oxm_view, out: *const oxm_view) -> c_int;
    pub fn oxm_batched_matmul(ctx: *mut oxm_ctx, a: *const oxm_view, b: *const oxm_view, out: *const oxm_view) -> c_int;
    pub fn oxm_matmul_fused(ctx: *mut oxm_ctx, a: *const oxm_view, b: *const oxm_view, out: *const oxm_view, ep: *const oxm_epilogue) -> c_int;
    pub fn oxm_matmul_mx(ctx: *mut oxm_ctx, a: *const oxm_view, a_scale: *const oxm_view, b: *const oxm_view, b_scale: *const oxm_view, out: *const oxm_view) -> c_int;
    pub fn oxm_unary(ctx: *mut oxm_ctx, op: c_int, a: *const oxm_view, out: *const oxm_view) -> c_int;
    pub fn oxm_binary(ctx: *mut oxm_ctx, op: c_int, a: *const oxm_view, b: *const oxm_view, out: *const oxm_view) -> c_int;
    pub fn oxm_reduce(ctx: *mut oxm_ctx, op: c_int, a: *const oxm_view, axes: *const i32, naxes: c_int, out: *const oxm_view) -> c_int;
    pub fn oxm_batched_matmul_host(ctx: *mut oxm_ctx, a: *const oxm_view, b: *const oxm_view, out: *const oxm_view) -> c_int;
    pub fn oxm_matmul_f32_noalloc(ctx: *mut oxm_ctx, a: *const oxm_view, b: *const oxm_view, out: *const oxm_view) -> c_int;
    pub fn oxm_contiguous(ctx: *mut oxm_ctx, src: *const oxm_view, dst: *const oxm_view) -> c_int;

    // ---- instrumentation ----
    pub fn oxm_event_create(ctx: *mut oxm_ctx, out: *mut *mut oxm_event) -> c_int;
    pub fn oxm_event_destroy(ev: *mut oxm_event) -> c_int;
    pub fn oxm_event_record(ctx: *mut oxm_ctx, ev: *mut oxm_event) -> c_int;
    pub fn oxm_event_elapsed_ms(start: *mut oxm_event, stop: *mut oxm_event, ms: *mut c_float) -> c_int;
    pub fn oxm_stream_handle(ctx: *mut oxm_ctx, cuda_stream: *mut *mut c_void) -> c_int;
    pub fn oxm_fill(ctx: *mut oxm_ctx, dst_device: *mut c_void, dtype: c_int, n: i64, seed: u64, stream: u64, dist: c_int, scale: c_double) -> c_int;
    pub fn oxm_selftest_bounded_wait(ctx: *mut oxm_ctx, limit_ms: i64) -> c_int;
    pub fn oxm_set_option(ctx: *mut oxm_ctx, key: *const c_char, value: i64) -> c_int;
    pub fn oxm_get_option(ctx: *mut oxm_ctx, key: *const c_char, value: *mut i64) -> c_int;
    pub fn oxm_launch_counts(ctx: *mut oxm_ctx, counts: *mut i64) -> c_int;
    pub fn oxm_last_kernel(ctx: *mut oxm_ctx) -> *const c_char;
    pub fn oxm_memory_stats(ctx: *mut oxm_ctx, stats: *mut i64) -> c_int;
    pub fn oxm_plan_matmul(a: *const oxm_view, b: *const oxm_view, out: *const oxm_view, num_sms: c_int, plan: *mut i32) -> c_int;
}
