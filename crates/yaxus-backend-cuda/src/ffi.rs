//! UNVERIFIED: no rustc in the image this repository is built in; never compiled.
//!
//! The C ABI of libyaxus_cuda (`include/yaxus_cuda.h`), one declaration per header entry, in
//! the header's order.  `tests/test_abi.py` of the library's repository checks names and
//! argument counts against the header.
#![allow(non_camel_case_types, dead_code)]
use std::os::raw::{c_char, c_int, c_void};

pub const YX_PAGE: usize = 128;
pub const YX_HEAD_DIM: usize = 128;

pub const YX_OK: c_int = 0;
pub const YX_ERR_INVALID: c_int = 1;
pub const YX_ERR_CUDA: c_int = 2;
pub const YX_ERR_OOM: c_int = 3;
pub const YX_ERR_STATE: c_int = 4;
pub const YX_ERR_DEVICE: c_int = 5;
pub const YX_ERR_NCCL: c_int = 6;
pub const YX_ERR_UNSUPPORTED: c_int = 7;

pub const YX_F32: c_int = 0;
pub const YX_F16: c_int = 1;
pub const YX_BF16: c_int = 2;

pub const YX_STATIC_SPLITS: usize = 8;
pub const YX_STATIC_MAX_ROW_HEADS: usize = 1024;

#[repr(C)]
pub struct yx_ctx {
    _opaque: [u8; 0],
}
#[repr(C)]
pub struct yx_kv {
    _opaque: [u8; 0],
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct yx_rope {
    pub inv_freq: [f32; YX_HEAD_DIM / 2],
    pub concentration: f32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct yx_layer {
    pub window: i32,
    pub rope: yx_rope,
}

#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct yx_tuning {
    pub force_path: i32,
    pub ctas_per_sm: i32,
    pub share_prefix: i32,
    pub tile_min_rows: i32,
    pub cost32: i32,
    pub cost64: i32,
    pub stages: i32,
    pub share_rows: i32,
    pub item_cost: i32,
    pub fused_merge: i32,
    pub tile_single: i32,
    pub min_piece: i32,
    pub overlap_calls: i32,
}

#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct yx_plan_info {
    pub path: i32,
    pub n_ctas: i32,
    pub n_items: i32,
    pub n_parts: i32,
    pub tiles: i64,
    pub unique_kv_bytes: i64,
    pub logical_kv_bytes: i64,
    pub launches: i32,
    pub shared_groups: i32,
}

extern "C" {
    // ---- context
    pub fn yx_ctx_create(device: c_int, stream: *mut c_void, out: *mut *mut yx_ctx) -> c_int;
    pub fn yx_ctx_destroy(ctx: *mut yx_ctx);
    pub fn yx_status(ctx: *const yx_ctx) -> c_int;
    pub fn yx_last_error(ctx: *const yx_ctx) -> *const c_char;
    pub fn yx_clear_error(ctx: *mut yx_ctx);
    pub fn yx_sync(ctx: *mut yx_ctx) -> c_int;
    pub fn yx_stream(ctx: *const yx_ctx) -> *mut c_void;
    pub fn yx_set_tuning(ctx: *mut yx_ctx, tuning: *const yx_tuning) -> c_int;
    pub fn yx_last_plan(ctx: *const yx_ctx, out: *mut yx_plan_info) -> c_int;
    pub fn yx_launch_count(ctx: *const yx_ctx) -> i64;
    pub fn yx_profile_begin(ctx: *mut yx_ctx) -> c_int;
    pub fn yx_profile_end(ctx: *mut yx_ctx, split_ms: *mut f32, combine_ms: *mut f32, calls: *mut c_int) -> c_int;
    // ---- tensors
    pub fn yx_tensor_alloc(ctx: *mut yx_ctx, bytes: usize, out_dev: *mut *mut c_void) -> c_int;
    pub fn yx_tensor_free(ctx: *mut yx_ctx, dev: *mut c_void) -> c_int;
    pub fn yx_upload(ctx: *mut yx_ctx, dst_dev: *mut c_void, src_host: *const c_void, bytes: usize) -> c_int;
    pub fn yx_download(ctx: *mut yx_ctx, dst_host: *mut c_void, src_dev: *const c_void, bytes: usize, wait: c_int) -> c_int;
    pub fn yx_host_alloc(ctx: *mut yx_ctx, bytes: usize, out_host: *mut *mut c_void) -> c_int;
    pub fn yx_host_free(ctx: *mut yx_ctx, host: *mut c_void) -> c_int;
    // ---- KV storage
    pub fn yx_kv_create(ctx: *mut yx_ctx, n_layers: c_int, layers: *const yx_layer, pages: u32, hkv: c_int, head_dim: c_int, dtype: c_int, max_pos: u32, out: *mut *mut yx_kv) -> c_int;
    pub fn yx_kv_destroy(ctx: *mut yx_ctx, kv: *mut yx_kv);
    pub fn yx_kv_copy_page(ctx: *mut yx_ctx, kv: *mut yx_kv, src: u32, dst: u32) -> c_int;
    pub fn yx_kv_read_pages(ctx: *mut yx_ctx, kv: *mut yx_kv, layer: c_int, first_page: u32, n_pages: u32, k_host: *mut c_void, v_host: *mut c_void) -> c_int;
    pub fn yx_kv_write_pages(ctx: *mut yx_ctx, kv: *mut yx_kv, layer: c_int, first_page: u32, n_pages: u32, k_host: *const c_void, v_host: *const c_void) -> c_int;
    // ---- a pass
    pub fn yx_begin_pass(ctx: *mut yx_ctx, rows: u32, pos_host: *const u32, kv_slot_host: *const u32, pt_off_host: *const u32, pages_host: *const u32, n_pages: u32) -> c_int;
    pub fn yx_attention(ctx: *mut yx_ctx, kv: *mut yx_kv, layer: c_int, qkv_dev: *const f32, q_norm_dev: *const f32, k_norm_dev: *const f32, hq: c_int, eps: f32, out_dev: *mut f32) -> c_int;
    pub fn yx_kv_append(ctx: *mut yx_ctx, kv: *mut yx_kv, layer: c_int, k_rows_dev: *const c_void, v_rows_dev: *const c_void, src_dtype: c_int) -> c_int;
    pub fn yx_attend(ctx: *mut yx_ctx, kv: *mut yx_kv, layer: c_int, q_dev: *const c_void, q_dtype: c_int, hq: c_int, window: i64, out_dev: *mut c_void, out_dtype: c_int) -> c_int;
    // ---- split-key partials and their merge
    pub fn yx_attend_partial(ctx: *mut yx_ctx, kv: *mut yx_kv, layer: c_int, q_dev: *const c_void, q_dtype: c_int, hq: c_int, window: i64, key_lo: u64, key_hi: u64, m_dev: *mut f32, l_dev: *mut f32, o_dev: *mut f32) -> c_int;
    pub fn yx_lse_combine(ctx: *mut yx_ctx, n_parts: c_int, m_dev: *const f32, l_dev: *const f32, o_dev: *const f32, n: usize, out_dev: *mut c_void, out_dtype: c_int) -> c_int;
    // ---- keys split across GPUs
    pub fn yx_comm_unique_id(out_id128: *mut c_void) -> c_int;
    pub fn yx_comm_create(ctx: *mut yx_ctx, n_ranks: c_int, rank: c_int, id128: *const c_void) -> c_int;
    pub fn yx_comm_destroy(ctx: *mut yx_ctx) -> c_int;
    pub fn yx_attend_allgather(ctx: *mut yx_ctx, kv: *mut yx_kv, layer: c_int, q_dev: *const c_void, q_dtype: c_int, hq: c_int, window: i64, key_lo: u64, key_hi: u64, out_dev: *mut c_void, out_dtype: c_int) -> c_int;
    // ---- the other operators of the Backend trait
    pub fn yx_embed(ctx: *mut yx_ctx, table_bf16_dev: *const c_void, vocab: u32, h: u32, ids_host: *const u32, rows: u32, out_dev: *mut f32) -> c_int;
    pub fn yx_rmsnorm(ctx: *mut yx_ctx, x_dev: *const f32, w_dev: *const f32, rows: u32, cols: u32, offset: f32, eps: f32, out_dev: *mut f32) -> c_int;
    pub fn yx_add_norm(ctx: *mut yx_ctx, x_dev: *mut f32, delta_dev: *const f32, post_w_dev: *const f32, post_offset: f32, pre_w_dev: *const f32, pre_offset: f32, eps: f32, rows: u32, cols: u32, out_dev: *mut f32) -> c_int;
    pub fn yx_matmul(ctx: *mut yx_ctx, x_dev: *const f32, w_bf16_dev: *const c_void, rows: u32, n: u32, k: u32, out_dev: *mut f32) -> c_int;
    pub fn yx_matmul_glu(ctx: *mut yx_ctx, x_dev: *const f32, w_bf16_dev: *const c_void, rows: u32, n: u32, k: u32, out_dev: *mut f32) -> c_int;
    pub fn yx_swiglu(ctx: *mut yx_ctx, x_dev: *const f32, rows: u32, inner: u32, out_dev: *mut f32) -> c_int;
    pub fn yx_add_assign(ctx: *mut yx_ctx, a_dev: *mut f32, b_dev: *const f32, n: usize) -> c_int;
    pub fn yx_select_rows(ctx: *mut yx_ctx, x_dev: *const f32, src_rows: u32, cols: u32, rows_host: *const u32, n: u32, out_dev: *mut f32) -> c_int;
    pub fn yx_argmax_rows(ctx: *mut yx_ctx, logits_dev: *const f32, rows: u32, cols: u32, out_host: *mut u32) -> c_int;
    // ---- attention without allocation
    pub fn yx_attend_static(ctx: *mut yx_ctx, kv: *mut yx_kv, layer: c_int, q_dev: *const c_void, q_dtype: c_int, hq: c_int, window: i64, out_dev: *mut c_void, out_dtype: c_int) -> c_int;
}
