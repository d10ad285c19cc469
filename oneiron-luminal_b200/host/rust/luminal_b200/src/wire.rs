//! Serialiser for the graph wire format of include/lum_llir.h.
//!
//! A lowered graph is `StableGraph<LLIROp, ()>` (src/graph.rs:23) whose nodes are boxed trait objects; a foreign runtime
//! cannot receive those, so every node is flattened to its egglog term name plus the term's parameters in term order
//! (`EgglogOp::term()`, src/op.rs:133-152).  Nodes are written in topological order and refer to their inputs by index.
use crate::ffi::*;
use luminal::prelude::*;
use luminal::shape::Term;

/// One parameter of a term, in the order `EgglogOp::term()` lists them.
#[derive(Debug, Clone)]
pub enum WireParam {
    Expr(Expression),
    EList(Vec<Expression>),
    /// index (in the serialised order) of the node this input comes from; filled in by `serialize`
    Input(usize),
    IList(Vec<usize>),
    Int(i64),
    Float(f64),
    Str(String),
    Dtype(u32),
}

/// A node ready to be written: the term name and its parameters.
#[derive(Debug, Clone)]
pub struct WireNode {
    pub op: String,
    pub params: Vec<WireParam>,
}

pub fn dtype_code(d: DType) -> u32 {
    match d {
        DType::F32 => LUM_F32,
        DType::F16 => LUM_F16,
        DType::Bf16 => LUM_BF16,
        DType::Int => LUM_INT,
        DType::Bool => LUM_BOOL,
        DType::NvFp4 => LUM_NVFP4,
        DType::Mxfp4 => LUM_MXFP4,
        // DType::Q8_0 => LUM_Q8_0 once the variant exists upstream (the five places it must be added are listed in
        // the repository's integration notes); until then Q8_0 weights are declared as U8-like raw inputs and
        // recognised by the `TileMatmulQ8` term.
    }
}

struct Out(Vec<u8>);
impl Out {
    fn u32(&mut self, v: u32) { self.0.extend_from_slice(&v.to_le_bytes()); }
    fn i32(&mut self, v: i32) { self.0.extend_from_slice(&v.to_le_bytes()); }
    fn i64(&mut self, v: i64) { self.0.extend_from_slice(&v.to_le_bytes()); }
    fn f64(&mut self, v: f64) { self.0.extend_from_slice(&v.to_le_bytes()); }
    fn str(&mut self, s: &str) { self.u32(s.len() as u32); self.0.extend_from_slice(s.as_bytes()); }
    /// Reverse-Polish terms exactly as `Expression` stores them (src/shape/expression.rs:132-147).
    fn expr(&mut self, e: &Expression) {
        let terms = e.terms.read();
        self.u32(terms.len() as u32);
        for t in terms.iter() {
            let (kind, val) = match *t {
                Term::Num(n) => (LUM_T_NUM, n),
                Term::Var(c) => (LUM_T_VAR, c as i32),
                Term::Add => (LUM_T_ADD, 0),
                Term::Sub => (LUM_T_SUB, 0),
                Term::Mul => (LUM_T_MUL, 0),
                Term::Div => (LUM_T_DIV, 0),
                Term::CeilDiv => (LUM_T_CEILDIV, 0),
                Term::Mod => (LUM_T_MOD, 0),
                Term::Min => (LUM_T_MIN, 0),
                Term::Max => (LUM_T_MAX, 0),
                Term::And => (LUM_T_AND, 0),
                Term::Or => (LUM_T_OR, 0),
                Term::Gte => (LUM_T_GTE, 0),
                Term::Lt => (LUM_T_LT, 0),
            };
            self.u32(kind);
            self.i32(val);
        }
    }
}

/// Writes `nodes` (already in topological order, `Input` parameters holding indices into the same slice).
pub fn serialize(nodes: &[WireNode]) -> Vec<u8> {
    let mut o = Out(Vec::with_capacity(64 * nodes.len() + 12));
    o.u32(LUM_LLIR_MAGIC);
    o.u32(LUM_LLIR_VERSION);
    o.u32(nodes.len() as u32);
    for (k, n) in nodes.iter().enumerate() {
        o.str(&n.op);
        o.u32(n.params.len() as u32);
        for p in &n.params {
            match p {
                WireParam::Expr(e) => { o.u32(LUM_P_EXPR); o.expr(e); }
                WireParam::EList(es) => { o.u32(LUM_P_ELIST); o.u32(es.len() as u32); for e in es { o.expr(e); } }
                WireParam::Input(i) => { assert!(*i < k, "graph not in topological order"); o.u32(LUM_P_INPUT); o.u32(*i as u32); }
                WireParam::IList(is) => { o.u32(LUM_P_ILIST); o.u32(is.len() as u32); for i in is { assert!(*i < k); o.u32(*i as u32); } }
                WireParam::Int(v) => { o.u32(LUM_P_INT); o.i64(*v); }
                WireParam::Float(v) => { o.u32(LUM_P_FLOAT); o.f64(*v); }
                WireParam::Str(s) => { o.u32(LUM_P_STR); o.str(s); }
                WireParam::Dtype(d) => { o.u32(LUM_P_DTYPE); o.u32(*d); }
            }
        }
    }
    o.0
}
