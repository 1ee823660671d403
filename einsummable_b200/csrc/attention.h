// Fused attention chain (scores -> mask -> softmax -> P V) on the tensor cores: attention.cu.
#pragma once
#include <cuda_runtime.h>

#include "common.h"

namespace es {

// Throws es_error when the descriptor or the pointers cannot be served.
void check_attention(es_attention_t const& a, void const* out, void const* q, void const* k, void const* v,
                     void const* mask);

void launch_attention(es_attention_t const& a, cudaStream_t stream, void* out, void const* q, void const* k,
                      void const* v, void const* mask);

// Algorithmic work of one launch: Q, K, V read and O written once plus the mask; 2 flops per
// multiply-add of both contractions.
inline uint64_t attention_bytes(es_attention_t const& a)
{
    uint64_t const bh = (uint64_t)a.batch * a.heads;
    return 2 * (bh * a.head_dim * (2ull * a.rows + 2ull * a.keys) + (uint64_t)a.rows * a.keys);
}
inline uint64_t attention_flops(es_attention_t const& a)
{
    return 4ull * a.batch * a.heads * a.rows * a.keys * a.head_dim;
}

// 0 = fine; 0x11..0x16 = a bounded wait inside the kernel gave up (Q copy, K copy, scores MMA,
// P tile, V copy, P V MMA)
unsigned int read_and_clear_attention_error();

// Trace builds (-DES_B200_TRACE): copies the first `n` of the 512 clock samples of the traced CTA (see
// attention.cu); returns the number copied, -1 when the library was built without the trace.
int read_attention_trace(unsigned long long* out, int n);

} // namespace es
