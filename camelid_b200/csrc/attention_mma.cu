// bfloat16 attention over the paged cache with mma.sync tensor-core tiles, for decode steps
// (prefill runs the tcgen05 kernel of attention_tc.cu), with float softmax and float accumulation.
//
// One block handles up to 16 (token, head) pairs that share one kv head: `rows_per_tile`
// consecutive new tokens of one sequence times `heads_per_cta` query heads, which fill the
// 16 rows of an m16n8k16 MMA, so the grouped heads (and in prefill a few neighbouring
// tokens) reuse every key and value that is read. Keys are walked in tiles of 32; the four
// warps of a block take tiles round-robin, each with its own cp.async pipeline into padded
// shared memory, and merge their running (max, sum, output) at the end. A range of keys
// can also be split over gridDim.z; the partial results are merged by the block that
// finishes last (a ticket per column of blocks), or by attn_combine_kernel where no tickets
// are given. Decode steps normally run attn_decode_fused_kernel further down instead: one
// launch from the split sums of the q/k/v product to the attention output.
//
// It replaces attention_decode / attn_sk_* and attention_batched / flash_pref_*
// (src/cuda_resident.rs:1587, :2332-2487, :1994, :2523-2705); the arithmetic is the
// reference's (src/inference.rs:23945-24025): (q . k) * scale, running maximum,
// exp(score - max), probabilities times values.
//
// Values of cache rows beyond a sequence's length never count: their probability is exactly
// zero, and the kernel zeroes those rows of its shared-memory tile before multiplying.
#include "attention_common.cuh"

#define AM_WARPS 4
#define AM_TILE 32
#define AM_STAGES 3

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int HD>
__global__ void __launch_bounds__(AM_WARPS * 32)
attn_paged_mma_kernel(AttnParams p) {
    constexpr int LDS = HD + 8;                              // padded row: conflict-free ldmatrix
    constexpr int TILE_ELEMS = AM_TILE * LDS;
    constexpr int STAGE_ELEMS = 2 * TILE_ELEMS;              // keys, then values
    constexpr int KSTEPS = HD / 16, DTILES = HD / 8;
    constexpr int CHUNKS = HD / 8;                           // 16-byte chunks of a row
    extern __shared__ __align__(16) uint8_t smem_raw[];
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    pdl_launch_dependents();
    // The step's integer arrays and the keys and values of earlier steps do not depend on the
    // kernels just before this one: everything up to the first read of q or of a freshly
    // written cache row runs ahead of pdl_wait().

    const int tile = blockIdx.x;
    const int seq = p.tile_seq[tile];
    const int q0 = p.tile_q0[tile];
    const int kvh = blockIdx.y / p.head_chunks;
    const int chunk = blockIdx.y - kvh * p.head_chunks;
    const int split = blockIdx.z;
    const int start = p.seq_start[seq];
    const int n_new = p.seq_new[seq];
    const int row0 = p.seq_row0[seq];
    const int group = p.n_heads / p.n_kv_heads;
    const int hpc = p.heads_per_cta;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows_in_tile = min(p.rows_per_tile, n_new - q0);
    const int kend = start + q0 + rows_in_tile;                          // exclusive
    const int kbeg = p.window > 0 ? max(0, start + q0 - p.window + 1) : 0;
    const int t_first = kbeg / AM_TILE;
    const int t_last = (kend + AM_TILE - 1) / AM_TILE;                   // exclusive
    const int per = (t_last - t_first + p.n_splits - 1) / p.n_splits;
    const int t_beg = t_first + split * per;
    const int t_end = min(t_last, t_beg + per);

    // the two MMA rows of this thread: i = lane/4 and i + 8
    int pos_r[2], lo_r[2];
    bool valid_r[2];
    const bf16* q_r[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int i = (lane >> 2) + 8 * h;
        const int r_local = i / hpc;
        const int hg = chunk * hpc + (i - r_local * hpc);
        valid_r[h] = (r_local < rows_in_tile) && (hg < group);
        pos_r[h] = start + q0 + r_local;
        lo_r[h] = p.window > 0 ? max(0, pos_r[h] - p.window + 1) : 0;
        q_r[h] = (const bf16*)p.q + (size_t)(row0 + q0 + r_local) * p.q_stride + (size_t)(kvh * group + hg) * HD;
    }
    float m_r[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_r[2] = {0.f, 0.f};
    float o[DTILES][4];
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[dt][i] = 0.f;

    const bf16* kp = (const bf16*)p.k_pages;
    const bf16* vp = (const bf16*)p.v_pages;
    bf16* my_smem = smem + (size_t)warp * AM_STAGES * STAGE_ELEMS;
    const uint32_t my_smem_u32 = (uint32_t)__cvta_generic_to_shared(my_smem);

    // this warp's tiles: t_beg + warp, + 4, + 8, ...
    const int n_mine = (t_end - t_beg - warp + AM_WARPS - 1) / AM_WARPS;
    // page of each of this warp's tiles, looked up once: lane i keeps the page of tile i (mod 32)
    const int* table_row = p.block_table + (size_t)seq * p.max_blocks;
    int my_page = 0;
    if (lane < n_mine) my_page = table_row[((t_beg + warp + lane * AM_WARPS) * AM_TILE) / CML_PAGE];

    auto issue = [&](int t, int stage, int it_index) {
        int page = __shfl_sync(0xffffffffu, my_page, it_index & 31);
        if (it_index >= 32) page = table_row[(t * AM_TILE) / CML_PAGE];
        const size_t base = (((size_t)page * p.n_kv_heads + kvh) * CML_PAGE + (t * AM_TILE) % CML_PAGE) * HD;
        const uint32_t dst = my_smem_u32 + (uint32_t)stage * STAGE_ELEMS * 2;
        for (int c = lane; c < AM_TILE * CHUNKS; c += 32) {
            const int r = c / CHUNKS, cc = c - r * CHUNKS;
            cp_async16(dst + (uint32_t)(r * LDS + cc * 8) * 2, kp + base + (size_t)r * HD + cc * 8);
            cp_async16(dst + (uint32_t)(TILE_ELEMS + r * LDS + cc * 8) * 2, vp + base + (size_t)r * HD + cc * 8);
        }
    };

    // tiles that lie wholly in what the cache held before this step are fetched at once
    bool early[AM_STAGES - 1];
#pragma unroll
    for (int s = 0; s < AM_STAGES - 1; ++s) {
        const int t = t_beg + warp + s * AM_WARPS;
        early[s] = s < n_mine && (t + 1) * AM_TILE <= start;
        if (early[s]) issue(t, s, s);
    }
    pdl_wait();
#pragma unroll
    for (int s = 0; s < AM_STAGES - 1; ++s) {
        if (s < n_mine && !early[s]) issue(t_beg + warp + s * AM_WARPS, s, s);
        cp_async_commit();
    }
    // A fragments of Q (zero rows where there is no query)
    uint32_t qa[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
        const int c = ks * 16 + 2 * (lane & 3);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            qa[ks][h] = valid_r[h] ? *reinterpret_cast<const uint32_t*>(q_r[h] + c) : 0u;
            qa[ks][h + 2] = valid_r[h] ? *reinterpret_cast<const uint32_t*>(q_r[h] + c + 8) : 0u;
        }
    }
    const float scale = p.scale;
    for (int it = 0; it < n_mine; ++it) {
        const int t = t_beg + warp + it * AM_WARPS;
        cp_async_wait<AM_STAGES - 2>();
        __syncwarp();
        {   // keep the pipeline full
            const int nxt = it + AM_STAGES - 1;
            if (nxt < n_mine) issue(t_beg + warp + nxt * AM_WARPS, nxt % AM_STAGES, nxt);
            cp_async_commit();
        }
        const uint32_t ks_u32 = my_smem_u32 + (uint32_t)(it % AM_STAGES) * STAGE_ELEMS * 2;
        const uint32_t vs_u32 = ks_u32 + TILE_ELEMS * 2;
        if ((t + 1) * AM_TILE > kend) {
            // value rows past the end of the sequence: their probability is zero, make the
            // product zero too whatever the page holds
            bf16* vs = my_smem + (size_t)(it % AM_STAGES) * STAGE_ELEMS + TILE_ELEMS;
            const int first = kend - t * AM_TILE;
            for (int c = lane; c < (AM_TILE - first) * (HD / 2); c += 32) {
                const int r = first + c / (HD / 2), d = (c % (HD / 2)) * 2;
                *reinterpret_cast<uint32_t*>(vs + r * LDS + d) = 0u;
            }
            __syncwarp();
        }

        // S = Q K^T : 16 x 32
        float s[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
            for (int np = 0; np < 2; ++np) {          // pairs of 8-key tiles
                const int mat = lane >> 3, rr = lane & 7;
                const int key = np * 16 + (mat >> 1) * 8 + rr;
                const int d = ks * 16 + (mat & 1) * 8;
                uint32_t b0, b1, b2, b3;
                ldsm_x4(ks_u32 + (uint32_t)(key * LDS + d) * 2, b0, b1, b2, b3);
                mma_bf16(s[np * 2], qa[ks], b0, b1);
                mma_bf16(s[np * 2 + 1], qa[ks], b2, b3);
            }
        }
        // scale, mask, running maximum
        const int key_base = t * AM_TILE + 2 * (lane & 3);
        float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int h = i >> 1;
                const int key = key_base + nt * 8 + (i & 1);
                const bool in = valid_r[h] && key <= pos_r[h] && key >= lo_r[h];
                s[nt][i] = in ? s[nt][i] * scale : -CUDART_INF_F;
                mx[h] = fmaxf(mx[h], s[nt][i]);
            }
        float corr[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float mn = fmaxf(m_r[h], mx[h]);
            m_use[h] = (mn == -CUDART_INF_F) ? 0.f : mn;
            corr[h] = (m_r[h] == -CUDART_INF_F) ? 0.f : __expf(m_r[h] - m_use[h]);
            m_r[h] = mn;
            l_r[h] *= corr[h];
        }
#pragma unroll
        for (int dt = 0; dt < DTILES; ++dt) {
            o[dt][0] *= corr[0]; o[dt][1] *= corr[0];
            o[dt][2] *= corr[1]; o[dt][3] *= corr[1];
        }
        // probabilities as A fragments (two k-steps of 16 keys)
        uint32_t pa[2][4];
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            float e[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    e[j][i] = __expf(s[kk * 2 + j][i] - m_use[i >> 1]);
                    l_r[i >> 1] += e[j][i];
                }
            pa[kk][0] = pack_bf16(e[0][0], e[0][1]);
            pa[kk][1] = pack_bf16(e[0][2], e[0][3]);
            pa[kk][2] = pack_bf16(e[1][0], e[1][1]);
            pa[kk][3] = pack_bf16(e[1][2], e[1][3]);
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
            for (int dp = 0; dp < DTILES / 2; ++dp) {
                const int mat = lane >> 3, rr = lane & 7;
                const int key = kk * 16 + (mat & 1) * 8 + rr;
                const int d = dp * 16 + (mat >> 1) * 8;
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t(vs_u32 + (uint32_t)(key * LDS + d) * 2, b0, b1, b2, b3);
                mma_bf16(o[dp * 2], pa[kk], b0, b1);
                mma_bf16(o[dp * 2 + 1], pa[kk], b2, b3);
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 1);
        l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 2);
    }
    __syncthreads();                       // every warp is done with its stage buffers

    // merge the four warps: [warp][16 rows][HD + 2] floats in shared memory
    float* red = reinterpret_cast<float*>(smem_raw);
    constexpr int RW = HD + 2;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float* dst = red + ((size_t)warp * 16 + (lane >> 2) + 8 * h) * RW;
        if ((lane & 3) == 0) {
            dst[0] = m_r[h];
            dst[1] = l_r[h];
        }
#pragma unroll
        for (int dt = 0; dt < DTILES; ++dt) {
            dst[2 + dt * 8 + 2 * (lane & 3)] = o[dt][2 * h];
            dst[2 + dt * 8 + 2 * (lane & 3) + 1] = o[dt][2 * h + 1];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 16 * (HD / 2); idx += blockDim.x) {
        const int i = idx / (HD / 2), d = (idx - i * (HD / 2)) * 2;
        const int r_local = i / hpc;
        const int hg = chunk * hpc + (i - r_local * hpc);
        if (r_local >= rows_in_tile || hg >= group) continue;
        float M = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < AM_WARPS; ++w) M = fmaxf(M, red[((size_t)w * 16 + i) * RW]);
        float L = 0.f, a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int w = 0; w < AM_WARPS; ++w) {
            const float* src = red + ((size_t)w * 16 + i) * RW;
            const float wgt = (src[0] == -CUDART_INF_F) ? 0.f : __expf(src[0] - M);
            L += wgt * src[1];
            a0 += wgt * src[2 + d];
            a1 += wgt * src[2 + d + 1];
        }
        const int row = row0 + q0 + r_local;
        const int head = kvh * group + hg;
        if (p.n_splits == 1) {
            const float inv = 1.0f / L;
            bf16* dst = (bf16*)p.out + (size_t)row * p.out_stride + (size_t)head * HD + d;
            *reinterpret_cast<uint32_t*>(dst) = pack_bf16(a0 * inv, a1 * inv);
        } else {
            float* dst = p.partial + (((size_t)row * p.n_heads + head) * p.n_splits + split) * RW;
            if (d == 0) {
                dst[0] = M;
                dst[1] = L;
            }
            dst[2 + d] = a0;
            dst[2 + d + 1] = a1;
        }
    }
    if (p.n_splits == 1 || p.tickets == nullptr) return;

    // The block that finishes last among the splits of this (tile, kv head chunk) merges
    // their partial results, in split order, and writes the output: no second kernel.
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    int* ticket = p.tickets + (size_t)tile * gridDim.y + blockIdx.y;
    if (threadIdx.x == 0) is_last = (atomicAdd(ticket, 1) == p.n_splits - 1);
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int idx = threadIdx.x; idx < 16 * (HD / 2); idx += blockDim.x) {
        const int i = idx / (HD / 2), d = (idx - i * (HD / 2)) * 2;
        const int r_local = i / hpc;
        const int hg = chunk * hpc + (i - r_local * hpc);
        if (r_local >= rows_in_tile || hg >= group) continue;
        const int row = row0 + q0 + r_local;
        const int head = kvh * group + hg;
        const float* base = p.partial + ((size_t)row * p.n_heads + head) * p.n_splits * RW;
        float M = -CUDART_INF_F;
        for (int s = 0; s < p.n_splits; ++s) M = fmaxf(M, __ldcg(base + (size_t)s * RW));
        float L = 0.f, a0 = 0.f, a1 = 0.f;
        for (int s = 0; s < p.n_splits; ++s) {
            const float* src = base + (size_t)s * RW;
            const float ms = __ldcg(src);
            const float wgt = (ms == -CUDART_INF_F) ? 0.f : __expf(ms - M);
            L += wgt * __ldcg(src + 1);
            a0 += wgt * __ldcg(src + 2 + d);
            a1 += wgt * __ldcg(src + 2 + d + 1);
        }
        const float inv = 1.0f / L;
        bf16* dst = (bf16*)p.out + (size_t)row * p.out_stride + (size_t)head * HD + d;
        *reinterpret_cast<uint32_t*>(dst) = pack_bf16(a0 * inv, a1 * inv);
    }
    if (threadIdx.x == 0) *ticket = 0;         // ready for the next launch
}

// ------------------------------------------------------------------------------------
// Decode, one launch from the q/k/v product to the attention output. Row r is the one new
// token of a sequence; a cluster of n_splits blocks owns (row, kv head) and every block a
// range of the cached keys, walked as above. Each block first sums the split partial sums of
// the q/k/v product for its heads (in split order, rounded to bfloat16 as the product's own
// epilogue would have), rotates q, and block 0 of the cluster also rotates the new key,
// writes key and value to the cache and counts them as one more range of one key. The
// ranges are merged inside the cluster: every block writes (max, sum, output) of its range
// into the shared memory of block 0 (distributed shared memory) and arrives on the cluster
// barrier; block 0 alone waits, merges the ranges in block order and writes the output.
// No q buffer, no partial results in global memory, no tickets. Cache tiles lie unpadded in
// shared memory with their 16-byte chunks swizzled by row (conflict-free ldmatrix).
//
// Keys below the row's position were written by earlier steps, so their tiles are fetched
// before pdl_wait(); with a borrowed cache (write_kv 0) the row's own key is already in the
// cache, written earlier in this step, and its tile is fetched after the wait.
struct AdParams {
    const float* partial;       // [gsplits][rows][width] partial sums of the q/k/v product
    int gsplits;
    long split_stride;
    int width;
    const int* row_pos;
    const int* row_seq;
    const int* block_table;
    int max_blocks;
    bf16* k_pages;
    bf16* v_pages;
    const float* inv_freq;
    int rotary_dim;
    int n_heads, n_kv_heads, write_kv, window, n_splits;
    float scale;
    bf16* out;
    int out_stride;
};

template <int HD>
__global__ void __launch_bounds__(AM_WARPS * 32)
attn_decode_fused_kernel(AdParams p) {
    constexpr int LDS = HD + 8;                              // rows of q_s
    constexpr int TILE_ELEMS = AM_TILE * HD;                 // cache tiles: no padding, 16-byte chunks swizzled by row
    constexpr int STAGE_ELEMS = 2 * TILE_ELEMS;
    constexpr int KSTEPS = HD / 16, DTILES = HD / 8;
    constexpr int CHUNKS = HD / 8;
    constexpr int RW = HD + 2;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __shared__ __align__(16) bf16 q_s[16 * LDS];      // rotated q of the grouped heads, zero rows beyond
    __shared__ float kv_new[2][HD];                   // the row's own key and value, as the cache keeps them
    __shared__ float s_new[16];                       // their scores
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    pdl_launch_dependents();
    // Distributed shared memory may be touched only once every block of the cluster runs: each
    // block arrives here, at its start, and waits just before its first store into block 0.
    if (p.n_splits > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

    const int split = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = p.row_pos[r];
    const int seq = p.row_seq[r];
    const int group = p.n_heads / p.n_kv_heads;
    const int kend = p.write_kv ? pos : pos + 1;                      // keys read from the cache: [kbeg, kend)
    const int kbeg = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int t_first = kbeg / AM_TILE;
    const int t_last = (kend + AM_TILE - 1) / AM_TILE;
    const int per = (t_last - t_first + p.n_splits - 1) / p.n_splits;
    const int t_beg = t_first + split * per;
    const int t_end = min(t_last, t_beg + per);
    const bool own_key = p.write_kv && split == 0;                    // this block accounts for the row's own key

    const bf16* kp = p.k_pages;
    const bf16* vp = p.v_pages;
    bf16* my_smem = smem + (size_t)warp * AM_STAGES * STAGE_ELEMS;
    const uint32_t my_smem_u32 = (uint32_t)__cvta_generic_to_shared(my_smem);
    const int n_mine = (t_end - t_beg - warp + AM_WARPS - 1) / AM_WARPS;
    const int* table_row = p.block_table + (size_t)seq * p.max_blocks;
    int my_page = 0;
    if (lane < n_mine) my_page = table_row[((t_beg + warp + lane * AM_WARPS) * AM_TILE) / CML_PAGE];

    auto issue = [&](int t, int stage, int it_index) {
        int page = __shfl_sync(0xffffffffu, my_page, it_index & 31);
        if (it_index >= 32) page = table_row[(t * AM_TILE) / CML_PAGE];
        const size_t base = (((size_t)page * p.n_kv_heads + kvh) * CML_PAGE + (t * AM_TILE) % CML_PAGE) * HD;
        const uint32_t dst = my_smem_u32 + (uint32_t)stage * STAGE_ELEMS * 2;
        for (int c = lane; c < AM_TILE * CHUNKS; c += 32) {
            const int rr = c / CHUNKS, cc = c - rr * CHUNKS;
            const uint32_t at = (uint32_t)(rr * HD + ((cc ^ (rr & 7)) * 8)) * 2;
            cp_async16(dst + at, kp + base + (size_t)rr * HD + cc * 8);
            cp_async16(dst + TILE_ELEMS * 2 + at, vp + base + (size_t)rr * HD + cc * 8);
        }
    };
    // Every stage is filled before the first tile is used: a block has few tiles, and what is
    // in flight from the start is what hides the latency of the cache reads.
    bool early[AM_STAGES];
#pragma unroll
    for (int s = 0; s < AM_STAGES; ++s) {
        const int t = t_beg + warp + s * AM_WARPS;
        early[s] = s < n_mine && (p.write_kv || (t + 1) * AM_TILE <= pos);
        if (early[s]) issue(t, s, s);
    }
    // What the rotation needs besides the product is ready before the product is: the items of
    // this thread, the sine and cosine of its first two, and the place of the row in the cache.
    const int half = p.rotary_dim >> 1, tail = HD - p.rotary_dim;
    const int n_rot_units = group + (own_key ? 1 : 0);
    const int n_pairs = n_rot_units * half;
    const int n_items = n_pairs + n_rot_units * tail + (own_key ? HD : 0);
    auto unit_col = [&](int u) {
        return u < group ? (kvh * group + u) * HD : (u == group ? (p.n_heads + kvh) * HD : (p.n_heads + p.n_kv_heads + kvh) * HD);
    };
    auto item_of = [&](int it, int& u, int& d0, int& d1) {      // u < 0: no item
        u = -1; d0 = -1; d1 = -1;
        if (it >= n_items) return;
        if (it < n_pairs) {
            u = it / half;
            d0 = it - u * half;
            d1 = d0 + half;
            return;
        }
        it -= n_pairs;
        if (it < n_rot_units * tail) {
            u = it / tail;
            d0 = p.rotary_dim + (it - u * tail);
            return;
        }
        u = group + 1;                                          // the value: no rotation
        d0 = it - n_rot_units * tail;
    };
    float sn0[2] = {0.f, 0.f}, cs0[2] = {1.f, 1.f};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        int u, d0, d1;
        item_of(j * AM_WARPS * 32 + (int)threadIdx.x, u, d0, d1);
        if (d1 >= 0) sincosf((float)pos * p.inv_freq[d0], &sn0[j], &cs0[j]);
    }
    size_t own_row = 0;
    if (own_key) own_row = (((size_t)table_row[pos / CML_PAGE] * p.n_kv_heads + kvh) * CML_PAGE + pos % CML_PAGE) * HD;
    pdl_wait();
#pragma unroll
    for (int s = 0; s < AM_STAGES; ++s) {
        if (s < n_mine && !early[s]) issue(t_beg + warp + s * AM_WARPS, s, s);
        cp_async_commit();
    }

    for (int i = threadIdx.x; i < (16 - group) * LDS; i += blockDim.x) q_s[group * LDS + i] = __float2bfloat16_rn(0.f);
    // q of the grouped heads (and, in block 0, the row's key and value) from the product's partial
    // sums. Work items are pairs (d, d + half) of a rotated head and single dimensions that pass
    // through; a thread takes two items at a time and has all their loads in flight at once.
    for (int base = 0; base < n_items; base += 2 * AM_WARPS * 32) {
        const float* src[2][2];
        int unit[2], dim[2][2];
        float acc[2][2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            item_of(base + j * AM_WARPS * 32 + (int)threadIdx.x, unit[j], dim[j][0], dim[j][1]);
            const float* row = p.partial + (size_t)r * p.width + (unit[j] >= 0 ? unit_col(unit[j]) : 0);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                src[j][e] = row + max(dim[j][e], 0);
                acc[j][e] = 0.f;
            }
        }
        for (int s0 = 0; s0 < p.gsplits; s0 += 8) {
            float t[2][2][8];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e)
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        // every load is unconditional (of a valid place), so that none waits for another
                        const float v = src[j][e][(size_t)min(s0 + i, p.gsplits - 1) * p.split_stride];
                        t[j][e][i] = (dim[j][e] >= 0 && s0 + i < p.gsplits) ? v : 0.f;
                    }
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e)
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[j][e] += t[j][e][i];          // split order
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            if (unit[j] < 0) continue;
            const int u = unit[j];
            auto store = [&](int d, float y) {
                const bf16 yb = __float2bfloat16_rn(y);
                if (u < group) q_s[u * LDS + d] = yb;
                else {
                    kv_new[u - group][d] = __bfloat162float(yb);
                    ((u == group ? p.k_pages : p.v_pages) + own_row)[d] = yb;
                }
            };
            const float x0 = __bfloat162float(__float2bfloat16_rn(acc[j][0]));      // as the product's epilogue rounds
            if (dim[j][1] >= 0) {
                const float x1 = __bfloat162float(__float2bfloat16_rn(acc[j][1]));
                float sn = sn0[j], cs = cs0[j];
                if (base > 0) sincosf((float)pos * p.inv_freq[dim[j][0]], &sn, &cs);
                store(dim[j][0], x0 * cs - x1 * sn);
                store(dim[j][1], x0 * sn + x1 * cs);
            } else {
                store(dim[j][0], x0);
            }
        }
    }
    __syncthreads();
    if (own_key) {
        for (int i = warp; i < group; i += AM_WARPS) {
            float acc = 0.f;
            for (int d = lane; d < HD; d += 32) acc = fmaf(__bfloat162float(q_s[i * LDS + d]), kv_new[0][d], acc);
            acc = warp_sum(acc);
            if (lane == 0) s_new[i] = acc * p.scale;
        }
    }
    // A fragments of Q
    bool valid_r[2];
    uint32_t qa[KSTEPS][4];
#pragma unroll
    for (int h = 0; h < 2; ++h) valid_r[h] = ((lane >> 2) + 8 * h) < group;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
        const int c = ks * 16 + 2 * (lane & 3);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const bf16* qrow = q_s + ((lane >> 2) + 8 * h) * LDS;
            qa[ks][h] = *reinterpret_cast<const uint32_t*>(qrow + c);
            qa[ks][h + 2] = *reinterpret_cast<const uint32_t*>(qrow + c + 8);
        }
    }
    float m_r[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_r[2] = {0.f, 0.f};
    float o[DTILES][4];
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[dt][i] = 0.f;

    const float scale = p.scale;
    for (int it = 0; it < n_mine; ++it) {
        const int t = t_beg + warp + it * AM_WARPS;
        cp_async_wait<AM_STAGES - 1>();
        __syncwarp();
        const uint32_t ks_u32 = my_smem_u32 + (uint32_t)(it % AM_STAGES) * STAGE_ELEMS * 2;
        const uint32_t vs_u32 = ks_u32 + TILE_ELEMS * 2;
        if ((t + 1) * AM_TILE > kend) {
            // value rows at and past the end: their probability is zero, make the product zero
            // too whatever the page holds there
            bf16* vs = my_smem + (size_t)(it % AM_STAGES) * STAGE_ELEMS + TILE_ELEMS;
            const int first = kend - t * AM_TILE;
            for (int c = lane; c < (AM_TILE - first) * (HD / 2); c += 32)
                *reinterpret_cast<uint32_t*>(vs + first * HD + c * 2) = 0u;          // whole rows, whatever their swizzle
            __syncwarp();
        }
        float s[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                const int mat = lane >> 3, rr = lane & 7;
                const int key = np * 16 + (mat >> 1) * 8 + rr;
                const int d = ks * 16 + (mat & 1) * 8;
                uint32_t b0, b1, b2, b3;
                ldsm_x4(ks_u32 + (uint32_t)(key * HD + (((d >> 3) ^ (key & 7)) << 3)) * 2, b0, b1, b2, b3);
                mma_bf16(s[np * 2], qa[ks], b0, b1);
                mma_bf16(s[np * 2 + 1], qa[ks], b2, b3);
            }
        }
        const int key_base = t * AM_TILE + 2 * (lane & 3);
        float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int h = i >> 1;
                const int key = key_base + nt * 8 + (i & 1);
                const bool in = valid_r[h] && key < kend && key >= kbeg;
                s[nt][i] = in ? s[nt][i] * scale : -CUDART_INF_F;
                mx[h] = fmaxf(mx[h], s[nt][i]);
            }
        float corr[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float mn = fmaxf(m_r[h], mx[h]);
            m_use[h] = (mn == -CUDART_INF_F) ? 0.f : mn;
            corr[h] = (m_r[h] == -CUDART_INF_F) ? 0.f : __expf(m_r[h] - m_use[h]);
            m_r[h] = mn;
            l_r[h] *= corr[h];
        }
#pragma unroll
        for (int dt = 0; dt < DTILES; ++dt) {
            o[dt][0] *= corr[0]; o[dt][1] *= corr[0];
            o[dt][2] *= corr[1]; o[dt][3] *= corr[1];
        }
        uint32_t pa[2][4];
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            float e[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    e[j][i] = __expf(s[kk * 2 + j][i] - m_use[i >> 1]);
                    l_r[i >> 1] += e[j][i];
                }
            pa[kk][0] = pack_bf16(e[0][0], e[0][1]);
            pa[kk][1] = pack_bf16(e[0][2], e[0][3]);
            pa[kk][2] = pack_bf16(e[1][0], e[1][1]);
            pa[kk][3] = pack_bf16(e[1][2], e[1][3]);
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
            for (int dp = 0; dp < DTILES / 2; ++dp) {
                const int mat = lane >> 3, rr = lane & 7;
                const int key = kk * 16 + (mat & 1) * 8 + rr;
                const int d = dp * 16 + (mat >> 1) * 8;
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t(vs_u32 + (uint32_t)(key * HD + (((d >> 3) ^ (key & 7)) << 3)) * 2, b0, b1, b2, b3);
                mma_bf16(o[dp * 2], pa[kk], b0, b1);
                mma_bf16(o[dp * 2 + 1], pa[kk], b2, b3);
            }
        }
        {   // the stage is free again: the tile that takes it
            __syncwarp();
            const int nxt = it + AM_STAGES;
            if (nxt < n_mine) issue(t_beg + warp + nxt * AM_WARPS, it % AM_STAGES, nxt);
            cp_async_commit();
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 1);
        l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 2);
    }
    __syncthreads();                       // every warp is done with its stage buffers

    // merge the four warps (and the row's own key) into this block's range, and hand the range
    // to block 0 of the cluster: into its shared memory, beyond everything it still uses
    float* red = reinterpret_cast<float*>(smem_raw);
    float* ranges = reinterpret_cast<float*>(smem_raw + (size_t)AM_WARPS * AM_STAGES * STAGE_ELEMS * sizeof(bf16));   // [n_splits][group][RW]
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float* dst = red + ((size_t)warp * 16 + (lane >> 2) + 8 * h) * RW;
        if ((lane & 3) == 0) {
            dst[0] = m_r[h];
            dst[1] = l_r[h];
        }
#pragma unroll
        for (int dt = 0; dt < DTILES; ++dt) {
            dst[2 + dt * 8 + 2 * (lane & 3)] = o[dt][2 * h];
            dst[2 + dt * 8 + 2 * (lane & 3) + 1] = o[dt][2 * h + 1];
        }
    }
    __syncthreads();
    if (p.n_splits > 1) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");      // all blocks have started
    uint32_t to_block0;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                 : "=r"(to_block0) : "r"((uint32_t)__cvta_generic_to_shared(ranges + (size_t)split * group * RW)), "r"(0u));
    for (int idx = threadIdx.x; idx < group * (HD / 2); idx += blockDim.x) {
        const int i = idx / (HD / 2), d = (idx - i * (HD / 2)) * 2;
        float M = own_key ? s_new[i] : -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < AM_WARPS; ++w) M = fmaxf(M, red[((size_t)w * 16 + i) * RW]);
        float L = 0.f, a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int w = 0; w < AM_WARPS; ++w) {
            const float* src = red + ((size_t)w * 16 + i) * RW;
            const float wgt = (src[0] == -CUDART_INF_F) ? 0.f : __expf(src[0] - M);
            L += wgt * src[1];
            a0 += wgt * src[2 + d];
            a1 += wgt * src[2 + d + 1];
        }
        if (own_key) {
            const float wgt = __expf(s_new[i] - M);
            L += wgt;
            a0 += wgt * kv_new[1][d];
            a1 += wgt * kv_new[1][d + 1];
        }
        if (p.n_splits == 1) {
            const float inv = 1.0f / L;
            bf16* dst = p.out + (size_t)r * p.out_stride + (size_t)(kvh * group + i) * HD + d;
            *reinterpret_cast<uint32_t*>(dst) = pack_bf16(a0 * inv, a1 * inv);
        } else {
            const uint32_t at = to_block0 + (uint32_t)(i * RW) * 4u;
            if (d == 0) asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(at), "f"(M), "f"(L) : "memory");
            asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(at + 8u + (uint32_t)d * 4u), "f"(a0), "f"(a1) : "memory");
        }
    }
    if (p.n_splits == 1) return;
    // Every block arrives once its range is written; only block 0 waits, so the others are done.
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    if (split != 0) return;
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    for (int idx = threadIdx.x; idx < group * (HD / 2); idx += blockDim.x) {
        const int i = idx / (HD / 2), d = (idx - i * (HD / 2)) * 2;
        float M = -CUDART_INF_F;
        for (int s = 0; s < p.n_splits; ++s) M = fmaxf(M, ranges[((size_t)s * group + i) * RW]);
        float L = 0.f, a0 = 0.f, a1 = 0.f;
        for (int s = 0; s < p.n_splits; ++s) {
            const float* src = ranges + ((size_t)s * group + i) * RW;
            const float wgt = (src[0] == -CUDART_INF_F) ? 0.f : __expf(src[0] - M);
            L += wgt * src[1];
            a0 += wgt * src[2 + d];
            a1 += wgt * src[2 + d + 1];
        }
        const float inv = 1.0f / L;
        bf16* dst = p.out + (size_t)r * p.out_stride + (size_t)(kvh * group + i) * HD + d;
        *reinterpret_cast<uint32_t*>(dst) = pack_bf16(a0 * inv, a1 * inv);
    }
}

template <int HD>
static int launch_mma(const AttnParams& p, int n_tiles, int n_rows, cudaStream_t s) {
    constexpr size_t stage_bytes = (size_t)AM_WARPS * AM_STAGES * 2 * AM_TILE * (HD + 8) * sizeof(bf16);
    constexpr size_t red_bytes = (size_t)AM_WARPS * 16 * (HD + 2) * sizeof(float);
    constexpr size_t smem = stage_bytes > red_bytes ? stage_bytes : red_bytes;
    dim3 grid(n_tiles, p.n_kv_heads * p.head_chunks, p.n_splits);
    cudaError_t e = cml_allow_smem<attn_paged_mma_kernel<HD>>(smem);
    if (e != cudaSuccess) return (int)e;
    e = launch_pdl(attn_paged_mma_kernel<HD>, grid, dim3(AM_WARPS * 32), smem, s, p);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (p.n_splits > 1 && p.tickets == nullptr) {
        launch_pdl(attn_combine_kernel<bf16>, dim3(n_rows * p.n_heads), dim3(HD >= 128 ? 128 : 64), 0, s,
                   (const float*)p.partial, (bf16*)p.out, p.out_stride, p.n_heads, HD, p.n_splits);
        e = cudaGetLastError();
    }
    return (int)e;
}

// `tickets` (may be null): n_tiles * n_kv_heads * head_chunks ints, zero before the first call and left zero;
// with it the last block of each column merges the splits itself, without it a second kernel does.
// bfloat16 only; head_dim 64 or 128 (others take the float kernel); rows_per_tile * heads_per_cta <= 16.
// q rows and the output must be 4-byte aligned (even strides).
extern "C" int cml_attn_paged_mma(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                  const void* v_pages, const int* block_table, int max_blocks, const int* tile_seq,
                                  const int* tile_q0, int n_tiles, const int* seq_row0, const int* seq_start,
                                  const int* seq_new, int n_rows, int n_heads, int n_kv_heads, int head_dim,
                                  int rows_per_tile, int heads_per_cta, int head_chunks, int n_splits, int window,
                                  float scale, float* partial, int* tickets, void* stream) {
    if (n_tiles <= 0 || n_rows <= 0) return 0;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return CML_ERR_BAD_SIZE;
    const int block_rows = rows_per_tile * heads_per_cta;       // the 16 rows of an MMA at most
    if (block_rows > 16 || rows_per_tile < 1 || heads_per_cta < 1) return CML_ERR_BAD_SIZE;
    if (heads_per_cta * head_chunks < n_heads / n_kv_heads) return CML_ERR_BAD_SIZE;
    if (n_splits < 1 || (n_splits > 1 && partial == nullptr)) return CML_ERR_BAD_SIZE;
    if ((q_stride & 1) || (out_stride & 1) || ((uintptr_t)q & 3) || ((uintptr_t)out & 3)) return CML_ERR_BAD_ALIGN;
    if (((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15)) return CML_ERR_BAD_ALIGN;
    AttnParams p;
    p.q = q; p.q_stride = q_stride; p.out = out; p.out_stride = out_stride;
    p.k_pages = k_pages; p.v_pages = v_pages; p.block_table = block_table; p.max_blocks = max_blocks;
    p.tile_seq = tile_seq; p.tile_q0 = tile_q0; p.seq_row0 = seq_row0; p.seq_start = seq_start; p.seq_new = seq_new;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim;
    p.rows_per_tile = rows_per_tile; p.heads_per_cta = heads_per_cta; p.head_chunks = head_chunks;
    p.n_splits = n_splits; p.window = window; p.scale = scale; p.partial = partial; p.tickets = tickets; p.n_stages = 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 64) return launch_mma<64>(p, n_tiles, n_rows, s);
    if (head_dim == 128) return launch_mma<128>(p, n_tiles, n_rows, s);
    return CML_ERR_BAD_SIZE;
}

template <int HD>
static int launch_decode_fused(const AdParams& p, int rows, cudaStream_t s) {
    constexpr size_t stage_bytes = (size_t)AM_WARPS * AM_STAGES * 2 * AM_TILE * HD * sizeof(bf16);
    static_assert(stage_bytes >= (size_t)AM_WARPS * 16 * (HD + 2) * sizeof(float), "the warps' merge reuses the stages");
    const int group = p.n_heads / p.n_kv_heads;
    // the ranges of all blocks of a cluster land in block 0, beyond its stages
    const size_t smem = stage_bytes + (p.n_splits > 1 ? (size_t)p.n_splits * group * (HD + 2) * sizeof(float) : 0);
    if (smem + 8 * 1024 > 227 * 1024) return CML_ERR_BAD_SIZE;
    cudaError_t e = cml_allow_smem<attn_decode_fused_kernel<HD>>(smem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.n_splits, p.n_kv_heads, rows);
    cfg.blockDim = dim3(AM_WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.n_splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = cml_pdl_enabled() ? 2 : 1;
    e = cudaLaunchKernelEx(&cfg, attn_decode_fused_kernel<HD>, p);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// Decode attention straight from the partial sums of the q/k/v product (see attn_decode_fused_kernel).
// partial: float [gsplits][rows][width], columns q heads, k heads, v heads. Row r is one new token at
// position row_pos[r] of sequence row_seq[r]. n_splits 1..8: blocks of a cluster per (row, kv head).
// bfloat16 cache and output; head_dim 64 or 128; at most 16 query heads per kv head.
extern "C" int cml_attn_decode_fused(const float* partial, int gsplits, long split_stride, int width, int rows,
                                     const int* row_pos, const int* row_seq, const int* block_table, int max_blocks,
                                     void* k_pages, void* v_pages, const float* inv_freq, int rotary_dim, int n_heads,
                                     int n_kv_heads, int head_dim, int write_kv, int window, float scale, int n_splits,
                                     void* out, int out_stride, void* stream) {
    if (rows <= 0) return 0;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || n_heads / n_kv_heads > 16) return CML_ERR_BAD_SIZE;
    if (n_splits < 1 || n_splits > 8 || gsplits < 1 || rows > 65535 || n_kv_heads > 65535) return CML_ERR_BAD_SIZE;
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) return CML_ERR_BAD_SIZE;
    if (width < (n_heads + (write_kv ? 2 * n_kv_heads : 0)) * head_dim) return CML_ERR_BAD_SIZE;
    if ((out_stride & 1) || ((uintptr_t)out & 3)) return CML_ERR_BAD_ALIGN;
    if (((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15)) return CML_ERR_BAD_ALIGN;
    AdParams p;
    p.partial = partial; p.gsplits = gsplits; p.split_stride = split_stride; p.width = width;
    p.row_pos = row_pos; p.row_seq = row_seq; p.block_table = block_table; p.max_blocks = max_blocks;
    p.k_pages = (bf16*)k_pages; p.v_pages = (bf16*)v_pages; p.inv_freq = inv_freq; p.rotary_dim = rotary_dim;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.write_kv = write_kv; p.window = window; p.n_splits = n_splits;
    p.scale = scale; p.out = (bf16*)out; p.out_stride = out_stride;
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 64) return launch_decode_fused<64>(p, rows, s);
    if (head_dim == 128) return launch_decode_fused<128>(p, rows, s);
    return CML_ERR_BAD_SIZE;
}
