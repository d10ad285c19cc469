// Temperature / top-k / top-p sampling of rows of logits on the device (declarations; the kernel is in lum_sample.cu).
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

#include "lum_kernels.cuh"

namespace lum {

constexpr int kSampleMaxK = 256;      // candidates a draw is made from

// What a draw depends on besides the logits; lives in device memory so that captured graphs stay valid when it changes.
struct SampleParams {
    float temperature;     // > 0
    float top_p;           // (0, 1]; >= 1 keeps all top_k candidates
    int top_k;             // 1 .. kSampleMaxK
    int pad;
    unsigned long long seed;
};

struct SampleArgs {
    const float* logits; size_t row_stride; int M, vocab;
    const SampleParams* params;
    int seq0; const int* row_seq;         // sequence id of row m: row_seq ? row_seq[m] : seq0 + m
    const int* draw_pos;                  // stand-alone use: the draw counter of row m (the position of the token being drawn)
    int* out;                             // optional [M]: the draws
    // single-token step (the head kernel ran with its own bookkeeping switched off): log the draw, make it the next token, advance
    DecodeState* state; int* tokens_out;
    // batched step (argmax_rows ran with its bookkeeping switched off): the same per row
    int* row_tok; int* row_pos; int* log; const int* step; int max_steps;
};

cudaError_t sample_rows_prepare();      // once per device before the first launch, outside stream capture
cudaError_t launch_sample_rows(const SampleArgs& a, cudaStream_t st);

}  // namespace lum
