//! `luminal_b200`: Luminal's `Runtime` trait (src/op.rs:10-30) over the B200 C-ABI library of include/lum_b200.h.
//!
//! ```ignore
//! let mut cx = Graph::default();
//! let model = Llama::init(&mut cx);                              // examples/llama/src/model.rs:29-114
//! let logits = model.forward(input, token_ids, &kv_cache).output();
//! cx.build_search_space::<B200Runtime>();                        // src/graph.rs:216-283 — uses B200Runtime::Ops
//! let mut rt = cx.search(B200Runtime::initialize(B200Arg::device(0)), 10);   // src/graph.rs:285-573
//! rt.load_safetensors(&cx, "model.safetensors");                 // bf16 / f16 / f32 checkpoint -> Q8_0 on the GPU
//! rt.set_data(input, prompt_ids);                                // crates/luminal_cuda/src/runtime.rs:160-165
//! cx.set_dim('s', n); cx.set_dim('p', 0);
//! rt.execute(&cx.dyn_map);
//! let row = rt.get_f32(logits);                                  // last-row logits
//! let next = rt.decode_greedy(256);                              // 256 tokens without leaving the device
//! ```
//!
//! Layout: `ffi` — raw declarations, checked against the header by the repository's tests; `wire` — the byte format a lowered
//! graph crosses the C boundary in (include/lum_llir.h); `ops` — the op set handed to the search: the block ops' egglog
//! terms and rewrite rules come from `luminal_cuda`, extraction produces nodes that can be serialised, plus the Q8_0
//! matrix product this backend adds; `runtime` — `impl Runtime for B200Runtime` and the inherent methods user code calls.
pub mod ffi;
pub mod ops;
pub mod runtime;
pub mod wire;

pub use runtime::{B200Arg, B200Error, B200Runtime};
