// Rotary position encoding of q and k, fused with the write of k and v into the paged cache.
//
// Replaces rope_rotate / rope_batched (src/cuda_resident.rs:1545, :1949) and kv_scatter /
// kv_scatter_batched (:1569, :1975). The angle is position * frequency in float, its sine
// and cosine come from sincosf (no fast-math), and pairs are (i, i + rotary_dim/2): the
// split-half pairing of un-permuted weights (src/inference/rope.rs:489-524, pairing at
// :501-509). Dimensions at and beyond rotary_dim pass through unchanged.
//
// The row's position is absolute; its page is looked up in the block table of its sequence.
#include "common.cuh"

// One block per token row. The sines and cosines of the row's position are computed once, by
// the first rotary_dim / 2 threads, and serve every head; then the threads walk work items of
// 8 consecutive dimensions of a head: a rotated pair of chunks (d, d + half), a chunk that
// passes through, or a chunk of v on its way to the cache. Chunks move as 16-byte vectors when
// the sizes and addresses allow (VEC), else element by element.
template <typename T>
__device__ __forceinline__ void rope_load8(const T* p, float (&v)[8], bool vec) {
    if (vec) {
        if (sizeof(T) == 2) {
            const uint4 u = *reinterpret_cast<const uint4*>(p);
            const bf16* h = reinterpret_cast<const bf16*>(&u);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __bfloat162float(h[i]);
        } else {
            const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = to_f32(p[i]);
    }
}
template <typename T>
__device__ __forceinline__ void rope_store8(T* p, const float (&v)[8], bool vec) {
    if (vec) {
        if (sizeof(T) == 2) {
            uint4 u;
            bf16* h = reinterpret_cast<bf16*>(&u);
#pragma unroll
            for (int i = 0; i < 8; ++i) h[i] = __float2bfloat16_rn(v[i]);
            *reinterpret_cast<uint4*>(p) = u;
        } else {
            reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
            reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) p[i] = from_f32<T>(v[i]);
    }
}

template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ row_pos,
                                     const int* __restrict__ row_seq, const int* __restrict__ block_table,
                                     int max_blocks, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     const float* __restrict__ inv_freq, int rotary_dim, int n_heads,
                                     int n_kv_heads, int head_dim, int write_kv, int vec) {
    extern __shared__ float rot_table[];          // cos [half], then sin [half]
    const int r = blockIdx.x;
    const int half = rotary_dim >> 1;
    const int pos = row_pos[r];                // the step's integer arrays do not depend on the kernels before
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        rot_table[i] = cs;
        rot_table[half + i] = sn;
    }
    size_t cache_row = 0;
    if (write_kv) {
        const int page = block_table[(size_t)row_seq[r] * max_blocks + pos / CML_PAGE];
        cache_row = ((size_t)page * n_kv_heads * CML_PAGE + pos % CML_PAGE) * head_dim;
    }
    __syncthreads();
    pdl_wait();
    pdl_launch_dependents();
    // Items per head: rotated heads (q, then k) have half/8 pair items and (head_dim - rotary_dim)/8
    // pass-through items; v heads have head_dim/8 copy items. Sizes are multiples of 8 here;
    // the launcher sends other sizes to the element-wise kernel.
    const int pair_items = half >> 3, tail_items = (head_dim - rotary_dim) >> 3, rot_items = pair_items + tail_items;
    const int n_rot = n_heads + (write_kv ? n_kv_heads : 0);
    const int copy_items = head_dim >> 3;
    const int n_items = n_rot * rot_items + (write_kv ? n_kv_heads * copy_items : 0);
    T* row = qkv + (size_t)r * row_stride;
    for (int it = threadIdx.x; it < n_items; it += blockDim.x) {
        if (it < n_rot * rot_items) {
            const int unit = it / rot_items, j = it - unit * rot_items;
            T* src = row + (size_t)unit * head_dim;
            T* dst = src;                       // q is rotated in place
            if (unit >= n_heads)
                dst = k_pages + cache_row + (size_t)(unit - n_heads) * CML_PAGE * head_dim;
            float a[8], b[8], ya[8], yb[8];
            if (j < pair_items) {
                const int d = j * 8;
                rope_load8(src + d, a, vec != 0);
                rope_load8(src + d + half, b, vec != 0);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float cs = rot_table[d + i], sn = rot_table[half + d + i];
                    ya[i] = a[i] * cs - b[i] * sn;
                    yb[i] = a[i] * sn + b[i] * cs;
                }
                rope_store8(dst + d, ya, vec != 0);
                rope_store8(dst + d + half, yb, vec != 0);
            } else if (dst != src) {
                const int d = rotary_dim + (j - pair_items) * 8;
                rope_load8(src + d, a, vec != 0);
                rope_store8(dst + d, a, vec != 0);
            }
        } else {
            const int c = it - n_rot * rot_items;
            const int h = c / copy_items, d = (c - h * copy_items) * 8;
            float a[8];
            rope_load8(row + (size_t)(n_heads + n_kv_heads + h) * head_dim + d, a, vec != 0);
            rope_store8(v_pages + cache_row + (size_t)h * CML_PAGE * head_dim + d, a, vec != 0);
        }
    }
}

// Element by element, one warp per (row, head): takes every even rotary_dim and every head size.
template <typename T>
__global__ void rope_kv_write_elem_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ row_pos,
                                     const int* __restrict__ row_seq, const int* __restrict__ block_table,
                                     int max_blocks, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     const float* __restrict__ inv_freq, int rotary_dim, int n_heads,
                                     int n_kv_heads, int head_dim, int write_kv) {
    pdl_wait();
    pdl_launch_dependents();
    // one warp per (row, head): q heads first, then k heads, then v heads
    const int r = blockIdx.x;
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int n_units = n_heads + (write_kv ? 2 * n_kv_heads : 0);
    if (unit >= n_units) return;
    const int half = rotary_dim >> 1;
    const int pos = row_pos[r];
    T* src = qkv + (size_t)r * row_stride + (size_t)unit * head_dim;
    T* dst = src;                               // q is rotated in place
    bool rotate = true;
    if (unit >= n_heads) {
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
            const float x0 = to_f32(src[i]), x1 = to_f32(src[i + half]);
            dst[i] = from_f32<T>(x0 * cs - x1 * sn);
            dst[i + half] = from_f32<T>(x0 * sn + x1 * cs);
        }
        if (dst != src)
            for (int d = rotary_dim + lane; d < head_dim; d += 32) dst[d] = src[d];
    } else {
        for (int d = lane; d < head_dim; d += 32) dst[d] = src[d];
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
            for (int i = 0; i < 8; ++i) {       // unconditional loads of valid places: none waits for another
                const float tv = src[(size_t)min(s0 + i, n_splits - 1) * split_stride + d];
                t[i] = (s0 + i < n_splits) ? tv : 0.f;
            }
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
    if ((head_dim & 7) || (rotary_dim & 15)) {          // the chunked kernel works on 8 dimensions at a time
        const int n_units = n_heads + (write_kv ? 2 * n_kv_heads : 0);
        const dim3 egrid(rows, (n_units + 7) / 8), eblock(256);
        if (egrid.y > 65535) return CML_ERR_BAD_SIZE;
        if (dtype == CML_DTYPE_F32)
            launch_pdl(rope_kv_write_elem_kernel<float>, egrid, eblock, 0, s, (float*)qkv, row_stride, row_pos, row_seq,
                       block_table, max_blocks, (float*)k_pages, (float*)v_pages, inv_freq, rotary_dim, n_heads,
                       n_kv_heads, head_dim, write_kv);
        else if (dtype == CML_DTYPE_BF16)
            launch_pdl(rope_kv_write_elem_kernel<bf16>, egrid, eblock, 0, s, (bf16*)qkv, row_stride, row_pos, row_seq,
                       block_table, max_blocks, (bf16*)k_pages, (bf16*)v_pages, inv_freq, rotary_dim, n_heads,
                       n_kv_heads, head_dim, write_kv);
        else
            return CML_ERR_BAD_DTYPE;
        return cml_launch_status();
    }
    const size_t esz = dtype == CML_DTYPE_F32 ? 4 : 2;
    // 16-byte (bfloat16) or 2 x 16-byte (float) vectors: every chunk of 8 elements must start on 16 bytes
    const int vec = (((uintptr_t)qkv | (uintptr_t)k_pages | (uintptr_t)v_pages) % 16 == 0) && ((row_stride * esz) % 16 == 0);
    const dim3 grid(rows), block(256);
    const size_t smem = (size_t)rotary_dim * sizeof(float);
    if (dtype == CML_DTYPE_F32)
        launch_pdl(rope_kv_write_kernel<float>, grid, block, smem, s, (float*)qkv, row_stride, row_pos, row_seq, block_table,
                                                              max_blocks, (float*)k_pages, (float*)v_pages, inv_freq,
                                                              rotary_dim, n_heads, n_kv_heads, head_dim, write_kv, vec);
    else if (dtype == CML_DTYPE_BF16)
        launch_pdl(rope_kv_write_kernel<bf16>, grid, block, smem, s, (bf16*)qkv, row_stride, row_pos, row_seq, block_table,
                                                             max_blocks, (bf16*)k_pages, (bf16*)v_pages, inv_freq,
                                                             rotary_dim, n_heads, n_kv_heads, head_dim, write_kv, vec);
    else
        return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}
