// Argument block and launchers of the routed mixture-of-experts kernels (lum_moe.cu).
#pragma once
#include "lum_kernels.cuh"

namespace lum {

struct MoeArgs {
    // routing (moe_route): residual rows in, normalised rows + routing out
    const float* x; int x_ld;                 // [n_tokens][x_ld]
    const void* gain; int gain_kind; float eps;
    const void* router; const void* router_bias;   // [n_experts][hidden], [n_experts] (element type: gain_kind)
    float* xf;                                // [n_tokens][slot]: hidden normalised activations, then top_k expert ids (int), then top_k weights
    int slot;                                 // floats per token slot (a multiple of 4)
    int hidden, ffn, n_experts, top_k;
    // experts (moe_gate_up, moe_down)
    const float* xf_in;                       // the slots the experts read: xf itself, or what the dispatch exchange delivered
    int n_tokens;
    int expert0, n_local;                     // this rank holds experts [expert0, expert0 + n_local)
    const int8_t* gu_q; const __half* gu_s; const void* gu_bias;   // local experts' gate_up planes [n_local * 2 * ffn, hidden] and bias
    const int8_t* dn_q; const __half* dn_s; const void* dn_bias;   // local experts' down planes [n_local * hidden, ffn] and bias
    float* sw;                                // [n_tokens][top_k][ffn] scratch: the gated activations
    float* out; float* out_add; int out_ld;   // out_add != null: += into the residual stream; else out = this rank's share
    float limit;
    int use_pdl;
};

cudaError_t launch_moe_route(const MoeArgs& a, int n_tokens, cudaStream_t st);
cudaError_t launch_moe_experts(const MoeArgs& a, int sm_count, cudaStream_t st);      // moe_gate_up, then moe_down
cudaError_t launch_moe_combine(float* x, const float* parts, int n_parts, int part_ld, int H, cudaStream_t st);

}  // namespace lum
