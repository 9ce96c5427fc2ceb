//! NOT COMPILED IN THIS ENVIRONMENT.
//!
//! The `extern "C"` surface of `include/candle_b200.h` and `include/candle_b200_nccl.h`, one
//! declaration per entry point, in the style of candle-flash-attn/src/ffi.rs:3-51.  Device pointers
//! travel as `*const c_void`; `stream` is the `CUstream` of the candle device.
use core::ffi::{c_char, c_int, c_void};

pub const DTYPE_F32: c_int = 0;
pub const DTYPE_F16: c_int = 1;
pub const DTYPE_BF16: c_int = 2;
pub const ID_U8: c_int = 0;
pub const ID_U32: c_int = 1;
pub const ID_I64: c_int = 2;
pub const STATUS_INVALID_INDEX: i32 = 1;
pub const STATUS_WAIT_TIMEOUT: i32 = 2;
pub const ROPE_INTERLEAVED: c_int = 0;
pub const ROPE_HALF: c_int = 1;
pub const ROPE_THD: c_int = 2;

/// `cb200_status`: what only the device can see (a bad id, a bounded wait that ran out).
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct Cb200Status {
    pub code: i32,
    pub reserved: i32,
    pub position: i64,
    pub index: i64,
    pub size: i64,
}

extern "C" {
    pub fn cb200_version() -> c_int;
    pub fn cb200_last_error() -> *const c_char;

    pub fn cb200_rms_norm(x: *const c_void, residual: *const c_void, alpha: *const c_void, y: *mut c_void,
        sum_out: *mut c_void, rows: i64, cols: i32, eps: f32, dtype: c_int, flags: c_int, stream: *mut c_void) -> c_int;
    pub fn cb200_rms_norm_checked(x: *const c_void, residual: *const c_void, alpha: *const c_void, y: *mut c_void,
        sum_out: *mut c_void, rows: i64, cols: i32, eps: f32, dtype: c_int, flags: c_int, status: *mut Cb200Status,
        stream: *mut c_void) -> c_int;
    pub fn cb200_layer_norm(x: *const c_void, residual: *const c_void, gamma: *const c_void, beta: *const c_void,
        y: *mut c_void, sum_out: *mut c_void, rows: i64, cols: i32, eps: f32, dtype: c_int, flags: c_int,
        stream: *mut c_void) -> c_int;
    pub fn cb200_layer_norm_checked(x: *const c_void, residual: *const c_void, gamma: *const c_void,
        beta: *const c_void, y: *mut c_void, sum_out: *mut c_void, rows: i64, cols: i32, eps: f32, dtype: c_int,
        flags: c_int, status: *mut Cb200Status, stream: *mut c_void) -> c_int;
    pub fn cb200_layer_norm_slow(x: *const c_void, weight: *const c_void, bias: *const c_void, y: *mut c_void,
        rows: i64, cols: i32, eps: f32, dtype: c_int, remove_mean: c_int, stream: *mut c_void) -> c_int;
    pub fn cb200_softmax_last_dim(x: *const c_void, y: *mut c_void, rows: i64, cols: i32, dtype: c_int,
        stream: *mut c_void) -> c_int;
    pub fn cb200_rope(src: *const c_void, cos: *const c_void, sin: *const c_void, dst: *mut c_void, b: i64, h: i32,
        t: i32, d: i32, dtype: c_int, variant: c_int, stream: *mut c_void) -> c_int;

    pub fn cb200_index_select(src: *const c_void, ids: *const c_void, out: *mut c_void, left: i64, src_dim: i64,
        right: i64, n_ids: i64, elem_size: i32, id_dtype: c_int, status: *mut Cb200Status, stream: *mut c_void) -> c_int;
    pub fn cb200_embedding(table: *const c_void, ids: *const c_void, out: *mut c_void, vocab: i64, hidden: i32,
        n_ids: i64, dtype: c_int, id_dtype: c_int, status: *mut Cb200Status, stream: *mut c_void) -> c_int;
    pub fn cb200_dequantize(blocks: *const c_void, qtype: c_int, out: *mut c_void, k: i64, out_dtype: c_int,
        stream: *mut c_void) -> c_int;
    pub fn cb200_qembedding(qtable: *const c_void, qtype: c_int, ids: *const c_void, out: *mut c_void, vocab: i64,
        hidden: i32, n_ids: i64, out_dtype: c_int, id_dtype: c_int, vocab_begin: i64, vocab_end: i64,
        status: *mut Cb200Status, stream: *mut c_void) -> c_int;
    pub fn cb200_embedding_rms_norm(table: *const c_void, ids: *const c_void, alpha: *const c_void, y: *mut c_void,
        gathered: *mut c_void, vocab: i64, hidden: i32, n_ids: i64, eps: f32, dtype: c_int, id_dtype: c_int,
        flags: c_int, status: *mut Cb200Status, stream: *mut c_void) -> c_int;
    pub fn cb200_qembedding_rms_norm(qtable: *const c_void, qtype: c_int, ids: *const c_void, alpha: *const c_void,
        y: *mut c_void, gathered: *mut c_void, vocab: i64, hidden: i32, n_ids: i64, eps: f32, out_dtype: c_int,
        id_dtype: c_int, vocab_begin: i64, vocab_end: i64, flags: c_int, status: *mut Cb200Status,
        stream: *mut c_void) -> c_int;
    pub fn cb200_qembedding_rms_norm_owner(qtable: *const c_void, qtype: c_int, ids: *const c_void,
        alpha: *const c_void, dsts: *const *mut c_void, n_dsts: c_int, vocab: i64, hidden: i32, n_ids: i64, eps: f32,
        out_dtype: c_int, id_dtype: c_int, vocab_begin: i64, vocab_end: i64, flags: c_int, status: *mut Cb200Status,
        stream: *mut c_void) -> c_int;
    pub fn cb200_qembedding_rms_norm_row_owner(qtable: *const c_void, qtype: c_int, ids: *const c_void,
        alpha: *const c_void, dsts: *const *mut c_void, n_dsts: c_int, row_bounds: *const i64, vocab: i64, hidden: i32,
        n_ids: i64, eps: f32, out_dtype: c_int, id_dtype: c_int, vocab_begin: i64, vocab_end: i64, flags: c_int,
        status: *mut Cb200Status, stream: *mut c_void) -> c_int;
    pub fn cb200_qembedding_route_rows(qtable: *const c_void, qtype: c_int, ids: *const c_void,
        dsts: *const *mut c_void, n_dsts: c_int, row_bounds: *const i64, vocab: i64, hidden: i32, n_ids: i64,
        id_dtype: c_int, vocab_begin: i64, vocab_end: i64, status: *mut Cb200Status, stream: *mut c_void) -> c_int;
}

#[cfg(feature = "nccl")]
extern "C" {
    pub fn cb200_sharded_qembedding_rms_norm(comm: *mut c_void, qtable: *const c_void, qtype: c_int,
        ids: *const c_void, alpha: *const c_void, y: *mut c_void, scratch: *mut c_void, scratch_bytes: usize,
        vocab: i64, hidden: i32, n_ids: i64, eps: f32, out_dtype: c_int, id_dtype: c_int, vocab_begin: i64,
        vocab_end: i64, flags: c_int, status: *mut Cb200Status, stream: *mut c_void) -> c_int;
    pub fn cb200_sharded_qembedding_rms_norm_static(comm: *mut c_void, qtable: *const c_void, qtype: c_int,
        ids: *const c_void, alpha: *const c_void, y: *mut c_void, vocab: i64, hidden: i32, n_ids: i64, eps: f32,
        out_dtype: c_int, id_dtype: c_int, vocab_begin: i64, vocab_end: i64, flags: c_int, status: *mut Cb200Status,
        stream: *mut c_void) -> c_int;
}
