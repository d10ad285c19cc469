//! Raw declarations of include/lum_b200.h (and the enums of include/lum_llir.h it uses).
//!
//! Kept in the header's order, one Rust item per C item; tests/test_rust_shim.py parses both files and fails when a
//! function, an argument type, a struct field or an enum value differs.
#![allow(non_camel_case_types, dead_code)]

use std::os::raw::{c_char, c_void};

/// Opaque runtime handle (`typedef struct lum_rt lum_rt`).
#[repr(C)]
pub struct lum_rt {
    _private: [u8; 0],
}
/// Opaque safetensors handle (`typedef struct lum_st lum_st`).
#[repr(C)]
pub struct lum_st {
    _private: [u8; 0],
}

pub const LUM_OK: i32 = 0;
pub const LUM_E_INVALID: i32 = -1;
pub const LUM_E_CUDA: i32 = -2;
pub const LUM_E_UNSUPPORTED: i32 = -3;
pub const LUM_E_DEVICE: i32 = -4;
pub const LUM_E_NOMEM: i32 = -5;

// lum_dtype (include/lum_llir.h): the first seven mirror luminal::op::DType
pub const LUM_F32: u32 = 0;
pub const LUM_F16: u32 = 1;
pub const LUM_BF16: u32 = 2;
pub const LUM_INT: u32 = 3;
pub const LUM_BOOL: u32 = 4;
pub const LUM_NVFP4: u32 = 5;
pub const LUM_MXFP4: u32 = 6;
pub const LUM_Q8_0: u32 = 7;

// lum_param_tag
pub const LUM_P_EXPR: u32 = 1;
pub const LUM_P_ELIST: u32 = 2;
pub const LUM_P_INPUT: u32 = 3;
pub const LUM_P_ILIST: u32 = 4;
pub const LUM_P_INT: u32 = 5;
pub const LUM_P_FLOAT: u32 = 6;
pub const LUM_P_STR: u32 = 7;
pub const LUM_P_DTYPE: u32 = 8;

// lum_term_kind: the order of luminal::shape::Term
pub const LUM_T_NUM: u32 = 0;
pub const LUM_T_VAR: u32 = 1;
pub const LUM_T_ADD: u32 = 2;
pub const LUM_T_SUB: u32 = 3;
pub const LUM_T_MUL: u32 = 4;
pub const LUM_T_DIV: u32 = 5;
pub const LUM_T_CEILDIV: u32 = 6;
pub const LUM_T_MOD: u32 = 7;
pub const LUM_T_MIN: u32 = 8;
pub const LUM_T_MAX: u32 = 9;
pub const LUM_T_AND: u32 = 10;
pub const LUM_T_OR: u32 = 11;
pub const LUM_T_GTE: u32 = 12;
pub const LUM_T_LT: u32 = 13;

pub const LUM_LLIR_MAGIC: u32 = 0x52494C4C;
pub const LUM_LLIR_VERSION: u32 = 1;

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct lum_config {
    pub device: i32,
    pub use_graph: i32,
    pub use_pdl: i32,
    pub attn_splits: i32,
    pub use_mega: i32,
    pub prefill_min_rows: i32,
    pub wait_budget_ms: i32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct lum_model_desc {
    pub n_layers: i32,
    pub hidden: i32,
    pub n_q_heads: i32,
    pub n_kv_heads: i32,
    pub head_dim: i32,
    pub ffn: i32,
    pub vocab: i32,
    pub max_seq: i32,
    pub rms_eps: f32,
    pub rope_theta: f32,
    pub rope_style: i32,
    pub weight_dtype: u32,
    pub embed_dtype: u32,
    pub kv_dtype: u32,
    pub qk_norm: i32,
    pub tied_head: i32,
    pub max_new_tokens: i32,
    pub tp_size: i32,
    pub tp_rank: i32,
    pub max_batch: i32,
    pub sliding_window: i32,
    pub window_even_layers: i32,
    pub attn_sinks: i32,
    pub proj_bias: i32,
    pub yarn_factor: f32,
    pub yarn_beta_fast: f32,
    pub yarn_beta_slow: f32,
    pub yarn_orig_max_pos: f32,
    pub n_experts: i32,
    pub top_k: i32,
    pub swiglu_limit: f32,
    pub ep_size: i32,
    pub ep_rank: i32,
    pub kv_page_rows: i32,
    pub kv_pool_pages: i32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct lum_sampling {
    pub temperature: f32,
    pub top_p: f32,
    pub top_k: i32,
    pub reserved: i32,
    pub seed: u64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct lum_stats {
    pub tokens_executed: u64,
    pub kernel_launches: u64,
    pub weight_bytes_per_token: u64,
    pub kv_bytes_per_position: u64,
    pub launches_per_step: i32,
    pub reserved: i32,
    pub last_profile_usec: f64,
}

unsafe extern "C" {
    pub fn lum_config_default(cfg: *mut lum_config);
    pub fn lum_create(cfg: *const lum_config, out: *mut *mut lum_rt) -> i32;
    pub fn lum_destroy(rt: *mut lum_rt);
    pub fn lum_last_error(rt: *const lum_rt) -> *const c_char;
    pub fn lum_device_info(rt: *const lum_rt, sm_count: *mut i32, mem_bytes: *mut u64, cc: *mut i32) -> i32;

    pub fn lum_model_init(rt: *mut lum_rt, desc: *const lum_model_desc) -> i32;
    pub fn lum_model_set_weight(rt: *mut lum_rt, slot: i32, layer: i32, data: *const c_void, bytes: usize, dtype: u32) -> i32;
    pub fn lum_model_set_weight_shard(rt: *mut lum_rt, slot: i32, layer: i32, data: *const c_void, bytes: usize, dtype: u32) -> i32;
    pub fn lum_load_safetensors(rt: *mut lum_rt, path: *const c_char, n_loaded: *mut i32, n_ignored: *mut i32) -> i32;
    pub fn lum_save_safetensors(rt: *mut lum_rt, path: *const c_char) -> i32;
    pub fn lum_model_synth(rt: *mut lum_rt, seed: u64) -> i32;
    pub fn lum_model_get_weight_f32(rt: *mut lum_rt, slot: i32, layer: i32, offset: usize, n: usize, host_out: *mut f32) -> i32;
    pub fn lum_model_weight_bytes(rt: *const lum_rt, bytes: *mut u64) -> i32;

    pub fn lum_llir_describe(blob: *const u8, size: usize, desc_out: *mut lum_model_desc, token_input: *mut i64, pos_input: *mut i64, logits_output: *mut i64, err: *mut c_char, err_len: usize) -> i32;
    pub fn lum_load_llir(rt: *mut lum_rt, blob: *const u8, size: usize, max_seq: i32, kv_dtype: u32, max_new_tokens: i32) -> i32;
    pub fn lum_set_input(rt: *mut lum_rt, hlir_node: i64, host: *const c_void, bytes: usize, dtype: u32) -> i32;
    pub fn lum_get_output(rt: *mut lum_rt, hlir_node: i64, host_out: *mut f32, n: usize) -> i32;
    pub fn lum_get_output_raw(rt: *mut lum_rt, hlir_node: i64, host_out: *mut c_void, capacity_bytes: usize, dtype: *mut u32, n_elems: *mut usize) -> i32;
    pub fn lum_set_input_device_ptr(rt: *mut lum_rt, hlir_node: i64, device_ptr: *const c_void, bytes: usize, dtype: u32) -> i32;

    pub fn lum_alloc_dummy_input(rt: *mut lum_rt, hlir_node: i64, n_elems: usize) -> i32;
    pub fn lum_clear_intermediates(rt: *mut lum_rt) -> i32;
    pub fn lum_profile_llir(rt: *mut lum_rt, blob: *const u8, size: usize, s: u64, p: u64, trials: i32, usec_per_execute: *mut f64, display: *mut c_char, display_len: usize) -> i32;
    pub fn lum_llir_describe_chunk(blob: *const u8, size: usize, desc_out: *mut lum_model_desc, hidden_input: *mut i64, hidden_output: *mut i64, err: *mut c_char, err_len: usize) -> i32;

    pub fn lum_kv_reset(rt: *mut lum_rt) -> i32;
    pub fn lum_kv_read(rt: *mut lum_rt, layer: i32, kind: i32, rows: i32, host_out: *mut f32) -> i32;
    pub fn lum_kv_save(rt: *mut lum_rt, layer: i32, kind: i32, rows: i32, host_out: *mut c_void, bytes: usize) -> i32;
    pub fn lum_kv_load(rt: *mut lum_rt, layer: i32, kind: i32, rows: i32, host: *const c_void, bytes: usize) -> i32;
    pub fn lum_kv_copy(rt: *mut lum_rt, src_seq: i32, dst_seq: i32, rows: i32) -> i32;
    pub fn lum_kv_release(rt: *mut lum_rt, seq: i32) -> i32;
    pub fn lum_kv_pool(rt: *const lum_rt, pages_total: *mut i32, pages_free: *mut i32, page_rows: *mut i32) -> i32;

    pub fn lum_set_dim(rt: *mut lum_rt, dim: c_char, value: u64) -> i32;
    pub fn lum_set_tokens(rt: *mut lum_rt, ids: *const i32, n: usize) -> i32;
    pub fn lum_execute(rt: *mut lum_rt) -> i32;
    pub fn lum_get_logits(rt: *mut lum_rt, host_out: *mut f32, n: usize) -> i32;
    pub fn lum_get_token(rt: *mut lum_rt, token: *mut i32) -> i32;
    pub fn lum_decode_greedy(rt: *mut lum_rt, n_steps: i32) -> i32;
    pub fn lum_get_decoded(rt: *mut lum_rt, host_out: *mut i32, n: usize) -> i32;
    pub fn lum_decode_reset(rt: *mut lum_rt) -> i32;
    pub fn lum_synchronize(rt: *mut lum_rt) -> i32;
    pub fn lum_set_sampling(rt: *mut lum_rt, s: *const lum_sampling) -> i32;

    pub fn lum_seq_select(rt: *mut lum_rt, seq: i32) -> i32;
    pub fn lum_batch_begin(rt: *mut lum_rt, n_seq: i32, tokens: *const i32, positions: *const i32) -> i32;
    pub fn lum_batch_begin_slots(rt: *mut lum_rt, n_seq: i32, slots: *const i32, tokens: *const i32, positions: *const i32) -> i32;
    pub fn lum_batch_decode(rt: *mut lum_rt, n_steps: i32) -> i32;
    pub fn lum_batch_get_decoded(rt: *mut lum_rt, host_out: *mut i32, n_steps: usize) -> i32;
    pub fn lum_batch_get_logits(rt: *mut lum_rt, seq: i32, host_out: *mut f32, n: usize) -> i32;

    pub fn lum_profile(rt: *mut lum_rt, trials: i32, usec_per_step: *mut f64, display: *mut c_char, display_len: usize) -> i32;
    pub fn lum_launches_per_step(rt: *const lum_rt, n: *mut i32) -> i32;
    pub fn lum_stream(rt: *mut lum_rt) -> *mut c_void;
    pub fn lum_get_stats(rt: *const lum_rt, out: *mut lum_stats) -> i32;
    pub fn lum_debug_wait_timeout(rt: *mut lum_rt) -> i32;

    pub fn lum_tp_unique_id(out128: *mut u8) -> i32;
    pub fn lum_tp_init(rt: *mut lum_rt, id128: *const u8, tp_size: i32, tp_rank: i32) -> i32;
    pub fn lum_tp_peer_export(rt: *mut lum_rt, handle64: *mut u8) -> i32;
    pub fn lum_tp_peer_import(rt: *mut lum_rt, handles: *const u8, n_ranks: i32) -> i32;

    pub fn lum_op_gemv_q8_0(quants_dev: *const i8, scales_dev: *const c_void, n: i32, k: i32, x_dev: *const f32, y_dev: *mut f32, force_direct: i32, stream: *mut c_void) -> i32;
    pub fn lum_q8_0_packed_bytes(n: i32, k: i32) -> usize;
    pub fn lum_op_q8_0_pack(quants_dev: *const i8, scales_dev: *const c_void, n: i32, k: i32, packed_dev: *mut c_void, stream: *mut c_void) -> i32;
    pub fn lum_op_gemv_q8_0_packed(packed_dev: *const c_void, n: i32, k: i32, x_dev: *const f32, y_dev: *mut f32, force_direct: i32, stream: *mut c_void) -> i32;
    pub fn lum_op_synth_q8_0_packed(seed: u64, tensor_id: u64, n: i32, k: i32, packed_dev: *mut c_void, stream: *mut c_void) -> i32;
    pub fn lum_op_gemm_q8_0_workspace(n: i32, k: i32, m: i32) -> usize;
    pub fn lum_op_gemm_q8_0_packed(packed_dev: *const c_void, n: i32, k: i32, x_dev: *const f32, m: i32, y_dev: *mut f32, workspace_dev: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> i32;
    pub fn lum_op_sample_q8_0(packed_dev: *const c_void, n: i32, k: i32, x_dev: *const f32, logits_dev: *mut f32, best_dev: *mut i32, stream: *mut c_void) -> i32;
    pub fn lum_op_sample_q8_0_static(packed_dev: *const c_void, n: i32, k: i32, x_dev: *const f32, logits_dev: *mut f32, best_dev: *mut i32, stream: *mut c_void) -> i32;
    pub fn lum_op_gemv_f32(w_dev: *const f32, n: i32, k: i32, x_dev: *const f32, y_dev: *mut f32, stream: *mut c_void) -> i32;
    pub fn lum_op_sample_topk(logits_dev: *const f32, n_rows: i32, vocab: i32, s: *const lum_sampling, seq0: i32, positions_dev: *const i32, tokens_dev: *mut i32, stream: *mut c_void) -> i32;
    pub fn lum_op_status(stream: *mut c_void) -> i32;
    pub fn lum_op_q8_0_quantize(src_dev: *const c_void, dtype: u32, n_elems: usize, quants_dev: *mut i8, scales_dev: *mut c_void, stream: *mut c_void) -> i32;

    pub fn lum_st_last_error() -> *const c_char;
    pub fn lum_st_open(path: *const c_char, out: *mut *mut lum_st) -> i32;
    pub fn lum_st_close(st: *mut lum_st);
    pub fn lum_st_count(st: *const lum_st) -> i32;
    pub fn lum_st_tensor(st: *const lum_st, i: i32, name: *mut *const c_char, dtype: *mut u32, ndim: *mut i32, shape8: *mut i64, data: *mut *const c_void, bytes: *mut usize) -> i32;
    pub fn lum_st_metadata(st: *const lum_st, key: *const c_char) -> *const c_char;
    pub fn lum_st_write(path: *const c_char, n: i32, names: *const *const c_char, dtypes: *const u32, ndims: *const i32, shapes8: *const i64, datas: *const *const c_void, n_meta: i32, meta_keys: *const *const c_char, meta_vals: *const *const c_char) -> i32;

    pub fn lum_op_q8_0_unpack(blocks_dev: *const u8, n_blocks: usize, quants_dev: *mut i8, scales_dev: *mut c_void, stream: *mut c_void) -> i32;
    pub fn lum_op_q8_0_dequant(quants_dev: *const i8, scales_dev: *const c_void, n_elems: usize, out_dev: *mut f32, stream: *mut c_void) -> i32;
    pub fn lum_op_synth_q8_0(seed: u64, tensor_id: u64, n_elems: usize, quants_dev: *mut i8, scales_dev: *mut c_void, stream: *mut c_void) -> i32;
    pub fn lum_op_synth_normal(seed: u64, tensor_id: u64, dtype: u32, n: usize, ones: i32, out_dev: *mut c_void, stream: *mut c_void) -> i32;
}
