//! The op set of this backend (`Runtime::Ops`).
//!
//! The search lowers HLIR to backend ops through each op's egglog term and rewrite rules (`EgglogOp::term / rewrites /
//! early_rewrites`, src/op.rs:133-152).  This backend wants the SAME lowering the CUDA backend's block ops describe — the
//! kernels behind the C ABI implement exactly that schedule — so every op here wraps the corresponding `luminal_cuda` op
//! and forwards `term`, `rewrites`, `early_rewrites` and `cleanup` to it.  What differs is `extract`: the CUDA backend
//! extracts into structs with private fields and generated kernel source; here extraction walks the term's parameter list
//! generically and produces a `WireNode` that can cross the C boundary.
//!
//! One op is new: `TileMatmulQ8`, a matrix product whose weight operand is Q8_0 (32 int8 quants + one f16 scale).  Its
//! parameter list is that of the reference's block-scaled products (`TileMatmulMxfp4`, crates/luminal_cuda/src/block/ops.rs:
//! 2388-2405) and its rule fires on the same Mul -> Sum shape with contiguous K on both operands, when the weight's dtype is Q8_0.
use std::fmt::Debug;
use std::marker::PhantomData;

use luminal::egglog_utils::{extract_dtype, extract_expr, extract_expr_list, SerializedEGraph};
use luminal::op::OpParam::{self, *};
use luminal::prelude::*;
use rustc_hash::FxHashMap;

use crate::wire::{dtype_code, WireNode, WireParam};

/// Dialect trait of this backend: every extracted op is a `WireNode` whose `Input` parameters still have to be resolved to
/// node indices (done by `B200Runtime::load_llir`, which knows the graph's edges).
pub trait B200Op: Debug {
    fn node(&self) -> &WireNode;
}

#[derive(Debug)]
pub struct Extracted(pub WireNode);
impl B200Op for Extracted {
    fn node(&self) -> &WireNode { &self.0 }
}

/// Generic extraction: one `WireParam` per entry of the term's parameter list; `Input` entries become the children the
/// search must extract next (their indices are patched in later, so a placeholder is stored).
fn extract_generic<'a>(
    name: &str,
    params: &[OpParam],
    egraph: &'a SerializedEGraph,
    children: &[&'a ENodeId],
    list_cache: &mut FxHashMap<&'a ENodeId, Vec<Expression>>,
    expr_cache: &mut FxHashMap<&'a ENodeId, Expression>,
) -> (LLIROp, Vec<&'a ENodeId>) {
    assert_eq!(params.len(), children.len(), "{name}: term arity and e-node children differ");
    let mut out = Vec::with_capacity(params.len());
    let mut inputs = Vec::new();
    let literal = |c: &ENodeId| egraph.enodes[c].0.replace('"', "");
    for (p, c) in params.iter().zip(children) {
        out.push(match p {
            EList => WireParam::EList(extract_expr_list(egraph, c, list_cache, expr_cache).unwrap()),
            Expr => WireParam::Expr(extract_expr(egraph, c, expr_cache).unwrap()),
            Input => { inputs.push(*c); WireParam::Input(usize::MAX) }
            IList => panic!("{name}: input lists are not used by this backend's ops"),
            Int => WireParam::Int(literal(c).parse().unwrap()),
            Float => WireParam::Float(literal(c).parse().unwrap()),
            Str => WireParam::Str(literal(c)),
            Dty => WireParam::Dtype(dtype_code(extract_dtype(egraph, c))),
        });
    }
    (LLIROp::new::<dyn B200Op>(Box::new(Extracted(WireNode { op: name.to_string(), params: out }))), inputs)
}

/// An op of the CUDA backend, re-extracted for this one.
#[derive(Debug, Default)]
pub struct Wrapped<D: EgglogOp + Default + Debug>(D, PhantomData<D>);

impl<D: EgglogOp + Default + Debug + 'static> EgglogOp for Wrapped<D> {
    fn term(&self) -> (String, Vec<OpParam>) { self.0.term() }
    fn rewrites(&self) -> Vec<String> { self.0.rewrites() }
    fn early_rewrites(&self) -> Vec<String> { self.0.early_rewrites() }
    fn cleanup(&self) -> bool { self.0.cleanup() }
    fn extract<'a>(
        &'a self,
        egraph: &'a SerializedEGraph,
        children: &[&'a ENodeId],
        list_cache: &mut FxHashMap<&'a ENodeId, Vec<Expression>>,
        expr_cache: &mut FxHashMap<&'a ENodeId, Expression>,
    ) -> (LLIROp, Vec<&'a ENodeId>) {
        let (name, params) = self.0.term();
        extract_generic(&name, &params, egraph, children, list_cache, expr_cache)
    }
}

/// Matrix product with a Q8_0 weight operand (the op this backend adds).
#[derive(Debug, Default)]
pub struct TileMatmulQ8;

impl EgglogOp for TileMatmulQ8 {
    fn term(&self) -> (String, Vec<OpParam>) {
        // sm_count, [M, N], m_tiles, n_tiles, K, a, a_m_stride, b, out_m_stride, out_n_stride
        ("TileMatmulQ8".to_string(), vec![Expr, EList, Expr, Expr, Expr, Input, Expr, Input, Expr, Expr])
    }
    fn cleanup(&self) -> bool { false }
    fn rewrites(&self) -> Vec<String> {
        // A broadcast product reduced over its last axis is a matrix product when K is contiguous in both operands and in the
        // reduction; it becomes this op when the right operand holds Q8_0 blocks.  Tile counts are informative only (the
        // kernels choose their own tiling): one row of tiles per 8 weight rows, one column per 32 activation rows.
        vec![r#"
        (rule
            ((= ?prod (Mul ?prod_shape ?x ?x_strides ?w ?w_strides ?prod_out_strides))
             (= ?acc (Sum ?out_shape ?k ?prod ?acc_in_strides ?acc_k_stride ?acc_out_strides))
             (= ?rows (nth_from_end ?out_shape 1))
             (= ?cols (nth_from_end ?out_shape 0))
             (!= ?rows (MNum 0))
             (!= ?cols (MNum 0))
             (= ?acc_k_stride (MNum 1))
             (= (nth_from_end ?x_strides 0) (MNum 1))
             (= (nth_from_end ?w_strides 0) (MNum 1))
             (= ?x_row_stride (nth_from_end ?x_strides 2))
             (= ?y_row_stride (nth_from_end ?acc_out_strides 1))
             (= ?y_col_stride (nth_from_end ?acc_out_strides 0))
             (= (Q8_0) (dtype ?w)))
            ((let ?mm (TileMatmulQ8 (MNum 148) ?out_shape (MCeilDiv ?rows (MNum 32)) (MCeilDiv ?cols (MNum 8)) ?k
                                    ?x ?x_row_stride ?w ?y_row_stride ?y_col_stride))
             (union ?acc ?mm)
             (set (dtype ?mm) (F32)))
            :name "q8_0 matrix product")
        "#.to_string()]
    }
    fn extract<'a>(
        &'a self,
        egraph: &'a SerializedEGraph,
        children: &[&'a ENodeId],
        list_cache: &mut FxHashMap<&'a ENodeId, Vec<Expression>>,
        expr_cache: &mut FxHashMap<&'a ENodeId, Expression>,
    ) -> (LLIROp, Vec<&'a ENodeId>) {
        let (name, params) = self.term();
        extract_generic(&name, &params, egraph, children, list_cache, expr_cache)
    }
}

use luminal_cuda::block as cb;
use luminal_cuda::kernel::hlir as ck;

/// What `Graph::build_search_space::<B200Runtime>()` registers: the logical ops, the block ops of the decoder schedule
/// (crates/luminal_cuda/src/block/ops.rs), the primitive fallbacks (crates/luminal_cuda/src/kernel/hlir.rs:53-69) — which the
/// library executes node by node when a graph has nothing else — and the Q8_0 product.
pub type Ops = (
    luminal_cuda::logical::Ops,
    (
        Wrapped<cb::RowAdd>, Wrapped<cb::RowSwishMul>, Wrapped<cb::RowRMSNorm>, Wrapped<cb::RowRope>, Wrapped<cb::RowEmbed>,
        Wrapped<cb::TileMatmulFullSplit>, TileMatmulQ8,
    ),
    (
        Wrapped<ck::KernelAdd>, Wrapped<ck::KernelMul>, Wrapped<ck::KernelMod>, Wrapped<ck::KernelLessThan>, Wrapped<ck::KernelIota>,
        Wrapped<ck::KernelGather>, Wrapped<ck::KernelSumReduce>, Wrapped<ck::KernelMaxReduce>, Wrapped<ck::KernelExp2>,
        Wrapped<ck::KernelLog2>, Wrapped<ck::KernelSin>, Wrapped<ck::KernelRecip>, Wrapped<ck::KernelSqrt>, Wrapped<ck::KernelConstant>,
        Wrapped<ck::KernelCast>,
    ),
);
