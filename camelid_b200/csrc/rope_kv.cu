// Rotary position encoding of q and k, fused with the write of k and v into the paged cache.
//
// Replaces rope_rotate / rope_batched (src/cuda_resident.rs:1545, :1949) and kv_scatter /
// kv_scatter_batched (:1569, :1975). The angle is position * frequency in float, its sine
// and cosine come from sincosf (no fast-math), and pairs are (i, i + rotary_dim/2): the
// split-half pairing of un-permuted weights (src/inference/rope.rs:489-524, pairing at
// :501-509). Dimensions at and beyond rotary_dim pass through unchanged.
//
// One block per token row. The row's position is absolute; its page is looked up in the
// block table of its sequence.
#include "common.cuh"

template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ row_pos,
                                     const int* __restrict__ row_seq, const int* __restrict__ block_table,
                                     int max_blocks, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     const float* __restrict__ inv_freq, int rotary_dim, int n_heads,
                                     int n_kv_heads, int head_dim, int write_kv) {
    extern __shared__ float sc[];              // cos[half], sin[half]
    pdl_wait();
    pdl_launch_dependents();
    const int half = rotary_dim >> 1;
    float* cs = sc;
    float* sn = sc + half;
    const int r = blockIdx.x;
    const int pos = row_pos[r];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float angle = (float)pos * inv_freq[i];
        float s, c;
        sincosf(angle, &s, &c);
        cs[i] = c;
        sn[i] = s;
    }
    __syncthreads();
    T* row = qkv + (size_t)r * row_stride;

    // q: rotate in place
    const int q_pairs = n_heads * half;
    for (int w = threadIdx.x; w < q_pairs; w += blockDim.x) {
        const int h = w / half, i = w - h * half;
        T* p = row + h * head_dim;
        const float x0 = to_f32(p[i]), x1 = to_f32(p[i + half]);
        p[i] = from_f32<T>(x0 * cs[i] - x1 * sn[i]);
        p[i + half] = from_f32<T>(x0 * sn[i] + x1 * cs[i]);
    }
    if (!write_kv) return;

    const int seq = row_seq[r];
    const int page = block_table[(size_t)seq * max_blocks + pos / CML_PAGE];
    const int in_page = pos % CML_PAGE;
    const T* ksrc = row + n_heads * head_dim;
    const T* vsrc = ksrc + n_kv_heads * head_dim;
    const size_t page_base = (size_t)page * n_kv_heads * CML_PAGE * head_dim;

    // k: rotate, then store; the pass-through dimensions are copied
    const int k_pairs = n_kv_heads * half;
    for (int w = threadIdx.x; w < k_pairs; w += blockDim.x) {
        const int h = w / half, i = w - h * half;
        const T* p = ksrc + h * head_dim;
        T* dst = k_pages + page_base + ((size_t)h * CML_PAGE + in_page) * head_dim;
        const float x0 = to_f32(p[i]), x1 = to_f32(p[i + half]);
        dst[i] = from_f32<T>(x0 * cs[i] - x1 * sn[i]);
        dst[i + half] = from_f32<T>(x0 * sn[i] + x1 * cs[i]);
    }
    const int tail = head_dim - rotary_dim;
    if (tail > 0) {
        for (int w = threadIdx.x; w < n_kv_heads * tail; w += blockDim.x) {
            const int h = w / tail, i = rotary_dim + (w - h * tail);
            k_pages[page_base + ((size_t)h * CML_PAGE + in_page) * head_dim + i] = ksrc[h * head_dim + i];
        }
    }
    // v: copy
    for (int w = threadIdx.x; w < n_kv_heads * head_dim; w += blockDim.x) {
        const int h = w / head_dim, i = w - h * head_dim;
        v_pages[page_base + ((size_t)h * CML_PAGE + in_page) * head_dim + i] = vsrc[w];
    }
}

// The same on the split sums of the q/k/v product: row r of the product is the sum over s of
// partial[s][r][:] (float, `width` columns, summed in index order) rounded to the compute
// type as the product's own epilogue would have. The rotated q goes to q_out in the compute
// type; k and v go to the cache. One warp per (row, head) so that a decode step of a few rows
// still spreads over many blocks.
template <typename T>
__global__ void rope_kv_from_partials_kernel(const float* __restrict__ partial, int n_splits, size_t split_stride,
                                             int width, T* __restrict__ q_out, int q_stride,
                                             const int* __restrict__ row_pos, const int* __restrict__ row_seq,
                                             const int* __restrict__ block_table, int max_blocks,
                                             T* __restrict__ k_pages, T* __restrict__ v_pages,
                                             const float* __restrict__ inv_freq, int rotary_dim, int n_heads,
                                             int n_kv_heads, int head_dim, int write_kv) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);    // q heads, then k heads, then v heads
    const int n_units = n_heads + (write_kv ? 2 * n_kv_heads : 0);
    if (unit >= n_units) return;
    const int half = rotary_dim >> 1;
    const int pos = row_pos[r];
    const float* src = partial + (size_t)r * width + (size_t)unit * head_dim;
    auto value = [&](int d) {          // loads of a group first, then the adds in split order
        float v = 0.f;
        for (int s0 = 0; s0 < n_splits; s0 += 8) {
            float t[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) t[i] = (s0 + i < n_splits) ? src[(size_t)(s0 + i) * split_stride + d] : 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) v += t[i];
        }
        return to_f32(from_f32<T>(v));
    };
    T* dst;
    bool rotate = true;
    if (unit < n_heads) {
        dst = q_out + (size_t)r * q_stride + (size_t)unit * head_dim;
    } else {
        const int seq = row_seq[r];
        const int page = block_table[(size_t)seq * max_blocks + pos / CML_PAGE];
        const int kv = unit - n_heads;
        const int h = kv < n_kv_heads ? kv : kv - n_kv_heads;
        rotate = kv < n_kv_heads;
        dst = (rotate ? k_pages : v_pages) + (((size_t)page * n_kv_heads + h) * CML_PAGE + pos % CML_PAGE) * head_dim;
    }
    if (rotate) {
        for (int i = lane; i < half; i += 32) {
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            const float x0 = value(i), x1 = value(i + half);
            dst[i] = from_f32<T>(x0 * cs - x1 * sn);
            dst[i + half] = from_f32<T>(x0 * sn + x1 * cs);
        }
        for (int d = rotary_dim + lane; d < head_dim; d += 32) dst[d] = from_f32<T>(value(d));
    } else {
        for (int d = lane; d < head_dim; d += 32) dst[d] = from_f32<T>(value(d));
    }
}

extern "C" int cml_rope_kv_from_partials(const float* partial, int n_splits, long split_stride, int width, void* q_out,
                                         int q_stride, int dtype, int rows, const int* row_pos, const int* row_seq,
                                         const int* block_table, int max_blocks, void* k_pages, void* v_pages,
                                         const float* inv_freq, int rotary_dim, int n_heads, int n_kv_heads,
                                         int head_dim, int write_kv, void* stream) {
    if (rows <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) return CML_ERR_BAD_SIZE;
    const int n_units = n_heads + (write_kv ? 2 * n_kv_heads : 0);
    if (width < n_units * head_dim) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(rows, (n_units + 3) / 4);
    if (grid.y > 65535) return CML_ERR_BAD_SIZE;
#define CML_RKP(T)                                                                                                    \
    launch_pdl(rope_kv_from_partials_kernel<T>, grid, dim3(128), 0, s, partial, n_splits, (size_t)split_stride, width, (T*)q_out,   \
                                                         q_stride, row_pos, row_seq, block_table, max_blocks,         \
                                                         (T*)k_pages, (T*)v_pages, inv_freq, rotary_dim, n_heads,     \
                                                         n_kv_heads, head_dim, write_kv)
    if (dtype == CML_DTYPE_F32) CML_RKP(float);
    else if (dtype == CML_DTYPE_BF16) CML_RKP(bf16);
    else return CML_ERR_BAD_DTYPE;
#undef CML_RKP
    return cml_launch_status();
}

extern "C" int cml_rope_kv_write(void* qkv, int dtype, int rows, int row_stride, const int* row_pos,
                                 const int* row_seq, const int* block_table, int max_blocks, void* k_pages,
                                 void* v_pages, const float* inv_freq, int rotary_dim, int n_heads,
                                 int n_kv_heads, int head_dim, int write_kv, void* stream) {
    if (rows <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)rotary_dim * sizeof(float);
    if (smem > 48 * 1024) return CML_ERR_BAD_SIZE;
    const int block = 256;
    if (dtype == CML_DTYPE_F32)
        launch_pdl(rope_kv_write_kernel<float>, dim3(rows), dim3(block), smem, s, (float*)qkv, row_stride, row_pos, row_seq, block_table,
                                                              max_blocks, (float*)k_pages, (float*)v_pages, inv_freq,
                                                              rotary_dim, n_heads, n_kv_heads, head_dim, write_kv);
    else if (dtype == CML_DTYPE_BF16)
        launch_pdl(rope_kv_write_kernel<bf16>, dim3(rows), dim3(block), smem, s, (bf16*)qkv, row_stride, row_pos, row_seq, block_table,
                                                             max_blocks, (bf16*)k_pages, (bf16*)v_pages, inv_freq,
                                                             rotary_dim, n_heads, n_kv_heads, head_dim, write_kv);
    else
        return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}
