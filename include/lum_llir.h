/*
 * lum_llir.h — wire format of a lowered graph ("LLIR") handed across the C ABI.
 *
 * In the reference the search hands a backend an in-process `LLIRGraph = StableGraph<LLIROp, ()>`
 * (src/graph.rs:23) through `Runtime::load_llir` (src/op.rs:16).  Each node was produced by an
 * op's `EgglogOp::extract`, whose fields are exactly the parameters of the op's egglog term
 * (`EgglogOp::term()`, src/op.rs:133-152; sorts in src/op.rs:298-322).  A foreign-language
 * runtime cannot receive boxed trait objects, so the same information is flattened into a byte
 * blob: one record per node, holding the term name and its parameters in term order.
 *
 * All integers little-endian.  Layout:
 *
 *   u32 magic = 0x52494C4C ("LLIR")   u32 version = 1   u32 n_nodes
 *   n_nodes x node:
 *       str  op            term name, e.g. "Input", "Add", "Sum", "RowRMSNorm", "TileMatmulQ8"
 *       u32  n_params
 *       n_params x param:  u32 tag, then
 *           LUM_P_EXPR   expr
 *           LUM_P_ELIST  u32 n, n x expr
 *           LUM_P_INPUT  u32 node index (must be < index of this node: nodes arrive toposorted)
 *           LUM_P_ILIST  u32 n, n x u32 node index
 *           LUM_P_INT    i64
 *           LUM_P_FLOAT  f64
 *           LUM_P_STR    str
 *           LUM_P_DTYPE  u32 (lum_dtype)
 *   str  = u32 byte length, bytes (no terminator, no padding)
 *   expr = u32 n_terms, n_terms x { u32 kind (lum_term_kind), i32 value }
 *
 * Expressions are the reference's reverse-Polish `Vec<Term>` (src/shape/expression.rs:132-147):
 * a binary term pops `a` then `b` and pushes `op(a, b)` — the FIRST popped value is the left
 * operand (src/shape/expression.rs:512-537).  `value` is the literal for LUM_T_NUM and the ASCII
 * code of the symbol for LUM_T_VAR ('z' is the loop variable, other letters are dynamic dims).
 *
 * Inputs of a node are its LUM_P_INPUT / LUM_P_ILIST parameters in order of appearance, which is
 * the reference's "incoming-edge insertion order" (crates/luminal_cuda/src/runtime.rs:525-529).
 */
#ifndef LUM_LLIR_H
#define LUM_LLIR_H

#include <stdint.h>

#define LUM_LLIR_MAGIC 0x52494C4Cu
#define LUM_LLIR_VERSION 1u

/* Element types; the first seven mirror `luminal::op::DType` (src/op.rs:161-182). LUM_Q8_0 is
 * the block format this runtime adds: 32 int8 quants sharing one binary16 scale. */
typedef enum lum_dtype {
    LUM_F32 = 0,
    LUM_F16 = 1,
    LUM_BF16 = 2,
    LUM_INT = 3,
    LUM_BOOL = 4,
    LUM_NVFP4 = 5,
    LUM_MXFP4 = 6,
    LUM_Q8_0 = 7
} lum_dtype;

typedef enum lum_param_tag {
    LUM_P_EXPR = 1,
    LUM_P_ELIST = 2,
    LUM_P_INPUT = 3,
    LUM_P_ILIST = 4,
    LUM_P_INT = 5,
    LUM_P_FLOAT = 6,
    LUM_P_STR = 7,
    LUM_P_DTYPE = 8
} lum_param_tag;

/* Same order as `enum Term` (src/shape/expression.rs:132-147). */
typedef enum lum_term_kind {
    LUM_T_NUM = 0,
    LUM_T_VAR = 1,
    LUM_T_ADD = 2,
    LUM_T_SUB = 3,
    LUM_T_MUL = 4,
    LUM_T_DIV = 5,
    LUM_T_CEILDIV = 6,
    LUM_T_MOD = 7,
    LUM_T_MIN = 8,
    LUM_T_MAX = 9,
    LUM_T_AND = 10,
    LUM_T_OR = 11,
    LUM_T_GTE = 12,
    LUM_T_LT = 13
} lum_term_kind;

/* Q8_0 wire block as this runtime accepts it through lum_set_input: the binary16 scale first,
 * then the 32 quants.  34 bytes, no padding.  (The reference has no Q8_0 code; the field order
 * is this library's own definition.) */
#define LUM_Q8_0_BLOCK 32
#define LUM_Q8_0_BLOCK_BYTES 34

#endif /* LUM_LLIR_H */
