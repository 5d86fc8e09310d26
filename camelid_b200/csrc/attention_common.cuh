// What the attention kernels share: the launch parameters and the merge of key ranges.
#pragma once
#include "common.cuh"
#include <math_constants.h>

struct AttnParams {
    const void* q;
    int q_stride;
    void* out;
    int out_stride;
    const void* k_pages;
    const void* v_pages;
    const int* block_table;
    int max_blocks;
    const int* tile_seq;
    const int* tile_q0;
    const int* seq_row0;
    const int* seq_start;
    const int* seq_new;
    int n_heads, n_kv_heads, head_dim;
    int rows_per_tile, heads_per_cta, head_chunks;
    int n_splits, window;
    float scale;
    float* partial;
    int* tickets;       // one zeroed counter per block column (tile, kv head chunk), or null
    int n_stages;       // float kernel: pages of keys and values a block keeps in shared memory (set by its launcher)
};

// Merge of the key ranges: out = sum_s exp(m_s - M) acc_s / sum_s exp(m_s - M) l_s, the
// ranges taken in index order. A range without visible keys has m = -inf and weight 0.
template <typename T>
__global__ void attn_combine_kernel(const float* __restrict__ partial, T* __restrict__ out, int out_stride,
                                    int n_heads, int head_dim, int n_splits) {
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x / n_heads, head = blockIdx.x - row * n_heads;
    const float* base = partial + (size_t)blockIdx.x * n_splits * (head_dim + 2);
    float M = -CUDART_INF_F;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, base[(size_t)s * (head_dim + 2)]);
    float L = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = base[(size_t)s * (head_dim + 2)];
        const float w = (ms == -CUDART_INF_F) ? 0.f : expf(ms - M);
        L += w * base[(size_t)s * (head_dim + 2) + 1];
    }
    const float inv = 1.0f / L;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float a = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = base[(size_t)s * (head_dim + 2)];
            const float w = (ms == -CUDART_INF_F) ? 0.f : expf(ms - M);
            a += w * base[(size_t)s * (head_dim + 2) + 2 + d];
        }
        out[(size_t)row * out_stride + head * head_dim + d] = from_f32<T>(a * inv);
    }
}

