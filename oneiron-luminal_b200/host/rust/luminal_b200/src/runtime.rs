//! `impl Runtime for B200Runtime` and the inherent methods user code calls on a runtime
//! (`set_data`, `get_f32`, `load_safetensors`; crates/luminal_cuda/src/runtime.rs:133-236).
use std::ffi::{c_void, CStr, CString};
use std::fmt;
use std::ptr;

use luminal::hlir::{Input, Output};
use luminal::prelude::*;
use petgraph::{algo::toposort, Direction};
use rustc_hash::FxHashMap;

use crate::ffi::*;
use crate::ops::B200Op;
use crate::wire::{dtype_code, serialize, WireNode, WireParam};

/// A failed call: the library's status code and message.  The reference panics in the same places and the search catches
/// the panic around a failing candidate (src/graph.rs:419-447); `check` below panics with this value for the same effect.
#[derive(Debug, Clone)]
pub struct B200Error {
    pub code: i32,
    pub message: String,
}
impl fmt::Display for B200Error {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result { write!(f, "[lum {}] {}", self.code, self.message) }
}
impl std::error::Error for B200Error {}

/// `Runtime::CompileArg`: which device, and the executor switches of `lum_config`.
#[derive(Debug, Clone, Copy)]
pub struct B200Arg {
    pub config: lum_config,
    /// KV-cache capacity in positions and its element type: caller-owned buffers in the reference (examples/llama/src/main.rs:19, 48),
    /// arguments of `lum_load_llir` here
    pub max_seq: i32,
    pub kv_dtype: u32,
    pub max_new_tokens: i32,
}
impl B200Arg {
    pub fn device(device: i32) -> Self {
        let mut config = lum_config::default();
        unsafe { lum_config_default(&mut config) };
        config.device = device;
        Self { config, max_seq: 4096, kv_dtype: LUM_BF16, max_new_tokens: 4096 }
    }
}

pub struct B200Runtime {
    h: *mut lum_rt,
    arg: B200Arg,
    /// what the loaded graph turned out to be (zeroed for a graph of primitive ops)
    desc: lum_model_desc,
    token_input: i64,
    logits_output: i64,
}

// one runtime = one device = one stream, used from one thread at a time (as the reference: crates/luminal_cuda/src/runtime.rs:123-130)
unsafe impl Send for B200Runtime {}

impl Drop for B200Runtime {
    fn drop(&mut self) { unsafe { lum_destroy(self.h) } }
}

impl B200Runtime {
    fn last_error(&self) -> String {
        unsafe { CStr::from_ptr(lum_last_error(self.h)) }.to_string_lossy().into_owned()
    }
    fn try_call(&self, rc: i32) -> Result<(), B200Error> {
        if rc == LUM_OK { Ok(()) } else { Err(B200Error { code: rc, message: self.last_error() }) }
    }
    /// Panics on failure, as the reference's runtime does; the context stays usable, so a caught panic loses nothing.
    fn check(&self, rc: i32) {
        if let Err(e) = self.try_call(rc) { panic!("{e}") }
    }

    /// Flattens a lowered graph: nodes in topological order, inputs by index, in incoming-edge insertion order
    /// (crates/luminal_cuda/src/runtime.rs:525-529).
    pub fn to_wire(graph: &LLIRGraph) -> Vec<u8> {
        let order = toposort(graph, None).expect("LLIR graph has a cycle");
        let index: FxHashMap<_, _> = order.iter().enumerate().map(|(i, n)| (*n, i)).collect();
        let mut nodes = Vec::with_capacity(order.len());
        for n in &order {
            // petgraph yields incoming edges newest first: reverse to get insertion order
            let mut srcs: Vec<usize> = graph.neighbors_directed(*n, Direction::Incoming).map(|s| index[&s]).collect();
            srcs.reverse();
            let op = &graph[*n];
            let node = if let Some(i) = op.to_op::<Input>() {
                WireNode { op: "Input".into(), params: vec![WireParam::Int(i.node as i64), WireParam::Str(i.label.clone()), WireParam::Dtype(dtype_code(i.dtype))] }
            } else if let Some(o) = op.to_op::<Output>() {
                WireNode { op: "Output".into(), params: vec![WireParam::Input(srcs[0]), WireParam::Int(o.node as i64)] }
            } else if let Some(b) = op.to_dialect::<dyn B200Op>() {
                let mut w = b.node().clone();
                let mut next = srcs.iter();
                for p in &mut w.params {
                    if let WireParam::Input(slot) = p { *slot = *next.next().expect("fewer edges than Input parameters"); }
                }
                w
            } else {
                panic!("op {op:?} is not part of the B200 op set");
            };
            nodes.push(node);
        }
        serialize(&nodes)
    }

    // ---- inherent methods, named as on `CudaRuntime` ---------------------------------------------------------------

    /// `set_data(id, data)` for i32 inputs (token ids): crates/luminal_cuda/src/runtime.rs:160-165
    pub fn set_data(&mut self, id: impl ToId, data: &[i32]) {
        let node = id.to_id().index() as i64;
        self.check(unsafe { lum_set_input(self.h, node, data.as_ptr() as *const c_void, data.len() * 4, LUM_INT) });
    }
    pub fn set_data_f32(&mut self, id: impl ToId, data: &[f32]) {
        let node = id.to_id().index() as i64;
        self.check(unsafe { lum_set_input(self.h, node, data.as_ptr() as *const c_void, data.len() * 4, LUM_F32) });
    }
    /// Q8_0 wire blocks (34 bytes per 32 weights) for a weight input
    pub fn set_data_q8_0(&mut self, id: impl ToId, blocks: &[u8]) {
        let node = id.to_id().index() as i64;
        self.check(unsafe { lum_set_input(self.h, node, blocks.as_ptr() as *const c_void, blocks.len(), LUM_Q8_0) });
    }
    /// The `CudaInput::Ptr` case (crates/luminal_cuda/src/runtime.rs:36-39): bytes already in device memory
    pub fn set_device_ptr(&mut self, id: impl ToId, device_ptr: u64, bytes: usize, dtype: DType) {
        let node = id.to_id().index() as i64;
        self.check(unsafe { lum_set_input_device_ptr(self.h, node, device_ptr as *const c_void, bytes, dtype_code(dtype)) });
    }

    /// `load_safetensors(cx, path)` (crates/luminal_cuda/src/runtime.rs:133-158).  The library matches tensor names to the decoder
    /// plan's slots (the labels the example models give their Inputs), converts or quantises on the GPU; `cx` is not needed.
    pub fn load_safetensors(&mut self, _cx: &Graph, path: &str) -> (i32, i32) {
        let p = CString::new(path).unwrap();
        let (mut loaded, mut ignored) = (0i32, 0i32);
        self.check(unsafe { lum_load_safetensors(self.h, p.as_ptr(), &mut loaded, &mut ignored) });
        (loaded, ignored)
    }
    pub fn save_shard(&mut self, path: &str) {
        let p = CString::new(path).unwrap();
        self.check(unsafe { lum_save_safetensors(self.h, p.as_ptr()) });
    }

    /// `get_f32(id)` (crates/luminal_cuda/src/runtime.rs:204-211): for a decoder, the last row of the logits
    pub fn get_f32(&self, id: impl ToId) -> Vec<f32> {
        let node = id.to_id().index() as i64;
        let mut n = if self.desc.vocab > 0 { (self.desc.vocab / self.desc.tp_size.max(1)) as usize } else { 0 };
        if n == 0 {
            self.check(unsafe { lum_get_output_raw(self.h, node, ptr::null_mut(), 0, ptr::null_mut(), &mut n) });
        }
        let mut out = vec![0f32; n];
        self.check(unsafe { lum_get_output(self.h, node, out.as_mut_ptr(), n) });
        out
    }
    /// `get_i32(id)` (crates/luminal_cuda/src/runtime.rs:220-226) for a graph of primitive ops
    pub fn get_i32(&self, id: impl ToId) -> Vec<i32> {
        let node = id.to_id().index() as i64;
        let (mut n, mut dt) = (0usize, 0u32);
        self.check(unsafe { lum_get_output_raw(self.h, node, ptr::null_mut(), 0, &mut dt, &mut n) });
        assert_eq!(dt, LUM_INT, "get_i32 on a tensor of another type");
        let mut out = vec![0i32; n];
        self.check(unsafe { lum_get_output_raw(self.h, node, out.as_mut_ptr() as *mut c_void, n * 4, ptr::null_mut(), ptr::null_mut()) });
        out
    }

    /// The sampled token of the last executed row (`sample`, examples/llama/src/main.rs:137-148, on the device)
    pub fn get_token(&self) -> i32 {
        let mut t = 0i32;
        self.check(unsafe { lum_get_token(self.h, &mut t) });
        t
    }
    /// `n` decode steps feeding each sample back in, without a host round trip per token (replaces the loop of
    /// examples/llama/src/main.rs:78-120); returns the tokens.
    pub fn decode_greedy(&mut self, n: usize) -> Vec<i32> {
        self.check(unsafe { lum_decode_reset(self.h) });
        self.check(unsafe { lum_decode_greedy(self.h, n as i32) });
        let mut out = vec![0i32; n];
        self.check(unsafe { lum_get_decoded(self.h, out.as_mut_ptr(), n) });
        out
    }
    pub fn kv_reset(&mut self) { self.check(unsafe { lum_kv_reset(self.h) }) }
    /// The sampler after the vocabulary projection; `None` = the greedy `sample` of examples/llama/src/main.rs:137-148.
    pub fn set_sampling(&mut self, s: Option<lum_sampling>) {
        let p = s.as_ref().map_or(std::ptr::null(), |v| v as *const lum_sampling);
        self.check(unsafe { lum_set_sampling(self.h, p) })
    }
    /// Several sequences side by side (`max_batch` cache slots): which slot `execute` addresses, a prefix copied between
    /// slots on the device, and batched steps over any set of live slots (row i works on `slots[i]`).
    pub fn seq_select(&mut self, seq: usize) { self.check(unsafe { lum_seq_select(self.h, seq as i32) }) }
    pub fn kv_copy(&mut self, src_seq: usize, dst_seq: usize, rows: usize) {
        self.check(unsafe { lum_kv_copy(self.h, src_seq as i32, dst_seq as i32, rows as i32) })
    }
    /// Paged cache (`kv_page_rows` > 0): a finished sequence's pages go back to the pool; (pages, free pages, rows per page).
    pub fn kv_release(&mut self, seq: usize) { self.check(unsafe { lum_kv_release(self.h, seq as i32) }) }
    pub fn kv_pool(&self) -> (i32, i32, i32) {
        let (mut a, mut b, mut c) = (0i32, 0i32, 0i32);
        self.check(unsafe { lum_kv_pool(self.h, &mut a, &mut b, &mut c) });
        (a, b, c)
    }
    pub fn batch_decode(&mut self, slots: &[i32], tokens: &[i32], positions: &[i32], n_steps: usize) -> Vec<i32> {
        assert!(slots.len() == tokens.len() && positions.len() == tokens.len(), "one entry per row in each list");
        self.check(unsafe { lum_batch_begin_slots(self.h, tokens.len() as i32, slots.as_ptr(), tokens.as_ptr(), positions.as_ptr()) });
        self.check(unsafe { lum_batch_decode(self.h, n_steps as i32) });
        let mut out = vec![0i32; n_steps * tokens.len()];
        self.check(unsafe { lum_batch_get_decoded(self.h, out.as_mut_ptr(), n_steps) });
        out
    }
    pub fn stats(&self) -> lum_stats {
        let mut s = lum_stats::default();
        self.check(unsafe { lum_get_stats(self.h, &mut s) });
        s
    }
    pub fn raw(&self) -> *mut lum_rt { self.h }
}

impl Runtime for B200Runtime {
    type Ops = crate::ops::Ops;
    type CompileArg = B200Arg;
    type ExecReturn = ();
    /// microseconds per execute, measured on the device
    type ProfileMetric = f64;

    fn initialize(arg: Self::CompileArg) -> Self {
        let mut h: *mut lum_rt = ptr::null_mut();
        let rc = unsafe { lum_create(&arg.config, &mut h) };
        if rc != LUM_OK {
            let msg = unsafe { CStr::from_ptr(lum_last_error(ptr::null())) }.to_string_lossy().into_owned();
            panic!("{}", B200Error { code: rc, message: msg });
        }
        Self { h, arg, desc: lum_model_desc::default(), token_input: -1, logits_output: -1 }
    }

    fn load_llir(&mut self, llir_graph: &LLIRGraph) {
        let blob = Self::to_wire(llir_graph);
        self.check(unsafe { lum_load_llir(self.h, blob.as_ptr(), blob.len(), self.arg.max_seq, self.arg.kv_dtype, self.arg.max_new_tokens) });
        // what the graph was recognised as (a graph of primitive ops describes nothing: the fields stay zero)
        let (mut tok, mut pos, mut out) = (-1i64, -1i64, -1i64);
        let mut d = lum_model_desc::default();
        let mut err = [0i8; 256];
        let rc = unsafe { lum_llir_describe(blob.as_ptr(), blob.len(), &mut d, &mut tok, &mut pos, &mut out, err.as_mut_ptr() as *mut _, err.len()) };
        if rc == LUM_OK { self.desc = d; self.token_input = tok; self.logits_output = out; } else { self.desc = lum_model_desc::default(); }
    }

    fn execute(&mut self, dyn_map: &FxHashMap<char, usize>) -> Self::ExecReturn {
        for (k, v) in dyn_map {
            self.check(unsafe { lum_set_dim(self.h, *k as std::os::raw::c_char, *v as u64) });
        }
        self.check(unsafe { lum_execute(self.h) });
    }

    fn profile(&mut self, llir_graph: &LLIRGraph, dyn_map: &FxHashMap<char, usize>, trials: usize) -> (Self::ProfileMetric, String) {
        let blob = Self::to_wire(llir_graph);
        let (s, p) = (*dyn_map.get(&'s').unwrap_or(&1) as u64, *dyn_map.get(&'p').unwrap_or(&0) as u64);
        let mut usec = 0f64;
        let mut text = [0i8; 160];
        self.check(unsafe { lum_profile_llir(self.h, blob.as_ptr(), blob.len(), s, p, trials as i32, &mut usec, text.as_mut_ptr() as *mut _, text.len()) });
        let display = unsafe { CStr::from_ptr(text.as_ptr() as *const _) }.to_string_lossy().into_owned();
        (usec, display)
    }

    fn allocate_dummy_input(&mut self, node_index: usize, num_elements: usize) {
        self.check(unsafe { lum_alloc_dummy_input(self.h, node_index as i64, num_elements) });
    }

    fn clear_intermediate_buffers(&mut self) {
        self.check(unsafe { lum_clear_intermediates(self.h) });
    }
}
