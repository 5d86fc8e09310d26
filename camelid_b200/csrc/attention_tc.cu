// Prefill attention on the fifth-generation tensor cores (bfloat16, head size 64 or 128).
//
// One block owns 128 (token, head) pairs of one kv head: 128 / heads_per_cta consecutive
// new tokens of one sequence times the grouped query heads, one pair per tensor-memory lane.
// Per page of 64 keys: S = Q K^T by tcgen05.mma into tensor memory; the 128 softmax threads
// each read their own row of S (no shuffles: a thread owns a row), keep the running maximum
// and sum in float, write the probabilities as bfloat16 into a swizzled shared-memory tile;
// P V by tcgen05.mma accumulates the output rows in a second tensor-memory buffer, which the
// same threads rescale in place on the rare pages where a row's reference maximum moves. Keys and values come straight from the cache pages by TMA (128-byte
// swizzle, no multicast); V is used as an MN-major operand, so no transpose is stored.
// MMA of the next page's S overlaps the softmax of this page; two blocks per SM (head size 64)
// overlap the rest: a softmax thread keeps its 64 scores and 32 packed probabilities in
// registers, and a third block per SM would make them spill. Blocks are numbered so that the
// tiles that see the most keys start first, for all kv heads alike.
//
// It replaces attention_batched / flash_pref_* (src/cuda_resident.rs:1994, :2523-2705);
// the arithmetic is the reference's (src/inference.rs:23945-24025): (q . k) * scale, running
// maximum, exp(score - max), probabilities times values.
//
// Warps 0-3: softmax (thread i = row i = tensor-memory lane i); warp 4: TMA producer;
// warp 5: tensor-memory allocation and MMA issue. Every mbarrier wait is bounded; on a
// timeout the kernel sets *err, lets its copies land, frees its tensor memory and returns.
#include "attention_common.cuh"
#include <cuda.h>

#define AT_ROWS 128
#define AT_KEYS 64
#define AT_STAGES 4
#define AT_THREADS 192
#define AT_WAIT_CYCLES 2000000000ll

struct AtParams {
    AttnParams a;
    int* err;
    int n_tiles;
};

__device__ __forceinline__ uint32_t at_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void at_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void at_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void at_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool at_mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool at_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (at_mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (at_mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > AT_WAIT_CYCLES) {
            *abort_flag = 1;
            return false;
        }
    }
}
__device__ __forceinline__ void at_tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ float at_max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ void at_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void at_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void at_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void at_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void at_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void at_ld16(uint32_t taddr, float* r) {
    uint32_t u[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
          "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = __uint_as_float(u[i]);
}

// 32 columns of this thread's lane, without waiting: several loads are issued, then one wait.
__device__ __forceinline__ void at_ld32_nowait(uint32_t taddr, float* r) {
    uint32_t* u = reinterpret_cast<uint32_t*>(r);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
          "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]),
          "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]),
          "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
        : "r"(taddr));
}
__device__ __forceinline__ void at_st32(uint32_t taddr, const float* r) {
    const uint32_t* u = reinterpret_cast<const uint32_t*>(r);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]), "r"(u[8]),
          "r"(u[9]), "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]), "r"(u[16]), "r"(u[17]),
          "r"(u[18]), "r"(u[19]), "r"(u[20]), "r"(u[21]), "r"(u[22]), "r"(u[23]), "r"(u[24]), "r"(u[25]), "r"(u[26]),
          "r"(u[27]), "r"(u[28]), "r"(u[29]), "r"(u[30]), "r"(u[31])
        : "memory");
}
__device__ __forceinline__ void at_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void at_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float at_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// K-major operand tile, rows of 128 bytes, 128-byte swizzle (as TMA writes it, and as the
// softmax threads write Q and P): stride 1024 bytes between groups of 8 rows.
__device__ __forceinline__ uint64_t at_desc_kmajor(uint32_t addr) {
    uint64_t d = (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// MN-major operand (V: rows are keys = K, 64 head dimensions contiguous per row, 128-byte
// swizzle): 8 keys per 1024-byte group (stride offset), blocks of 64 head dimensions
// `block_bytes` apart (leading offset).
__device__ __forceinline__ uint64_t at_desc_mnmajor(uint32_t addr, uint32_t block_bytes) {
    uint64_t d = (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((block_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a swizzled tile of 128-byte rows.
__device__ __forceinline__ uint32_t at_swizzled(int row, int chunk) {
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}

template <int HD>
__global__ void __launch_bounds__(AT_THREADS, HD == 64 ? 2 : 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV, AtParams ap) {
    const AttnParams& p = ap.a;
    constexpr int KB = HD / 64;                               // 64-column blocks of a head
    constexpr uint32_t Q_BYTES = AT_ROWS * 128 * KB;          // 16 KB per block
    constexpr uint32_t KV_BLOCK = AT_KEYS * 128;              // 8 KB: 64 keys x 64 dims
    constexpr uint32_t K_BYTES = KV_BLOCK * KB, V_BYTES = KV_BLOCK * KB;
    constexpr uint32_t P_BYTES = AT_ROWS * 128;
    constexpr uint32_t TMEM_COLS = HD == 64 ? 128 : 256;      // S: 64 columns, then P V: HD columns
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (at_smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - at_smem_u32(smem_raw));
    const uint32_t sQ = base, sP = sQ + Q_BYTES, sK = sP + P_BYTES, sV = sK + AT_STAGES * K_BYTES;
    const uint32_t bars = sV + AT_STAGES * V_BYTES;
    uint8_t* gQ = gbase;
    uint8_t* gP = gbase + Q_BYTES;
    uint8_t* gV = gbase + Q_BYTES + P_BYTES + AT_STAGES * K_BYTES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gbase + (bars - base) + 16 * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    auto kv_full = [&](int s) { return bars + 8u * s; };
    auto kv_empty = [&](int s) { return bars + 8u * (AT_STAGES + s); };
    const uint32_t s_full = bars + 8u * (2 * AT_STAGES), s_empty = s_full + 8, p_full = s_full + 16,
                   pv_full = s_full + 24, q_ready = s_full + 32;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 32) {      // the maps' own round trip, beside the set-up
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&mapK) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&mapV) : "memory");
    }
    // Blocks start in the order of blockIdx.x: the tiles that see the most keys come first, for
    // every kv head alike, so that no long tile starts late.
    const int n_cols = p.n_kv_heads * p.head_chunks;
    const int tile = ap.n_tiles - 1 - (int)(blockIdx.x / n_cols);
    const int col = (int)(blockIdx.x % n_cols);
    const int seq = p.tile_seq[tile];
    const int q0 = p.tile_q0[tile];
    const int kvh = col / p.head_chunks;
    const int chunk = col - kvh * p.head_chunks;
    const int start = p.seq_start[seq];
    const int n_new = p.seq_new[seq];
    const int row0 = p.seq_row0[seq];
    const int group = p.n_heads / p.n_kv_heads;
    const int hpc = p.heads_per_cta;
    const int rows_in_tile = min(p.rows_per_tile, n_new - q0);
    const int kend = start + q0 + rows_in_tile;
    const int kbeg = p.window > 0 ? max(0, start + q0 - p.window + 1) : 0;
    const int t_first = kbeg / AT_KEYS;
    const int n_tiles_k = (kend + AT_KEYS - 1) / AT_KEYS - t_first;

    if (threadIdx.x == 0) {
        for (int s = 0; s < AT_STAGES; ++s) {
            at_mbar_init(kv_full(s), 1);
            at_mbar_init(kv_empty(s), 1);
        }
        at_mbar_init(s_full, 1);
        at_mbar_init(s_empty, 128);
        at_mbar_init(p_full, 128);
        at_mbar_init(pv_full, 1);
        at_mbar_init(q_ready, 128);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        at_fence_async_smem();
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(at_smem_u32(tmem_slot)),
                     "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    at_fence_before();
    __syncthreads();
    at_fence_after();
    const uint32_t tmem_s = *tmem_slot;
    const uint32_t tmem_pv = tmem_s + 64;
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 4) {
        if (lane == 0) {
            const int* table_row = p.block_table + (size_t)seq * p.max_blocks;
            int issued = 0;
            for (int it = 0; it < n_tiles_k; ++it) {
                const int s = it % AT_STAGES;
                const uint32_t ph = (uint32_t)(it / AT_STAGES) & 1u;
                if (!at_mbar_wait(kv_empty(s), ph ^ 1u, abort_flag)) break;
                const int page = table_row[t_first + it];
                const int y = (page * p.n_kv_heads + kvh) * CML_PAGE;
                at_mbar_expect_tx(kv_full(s), K_BYTES + V_BYTES);
#pragma unroll
                for (int b = 0; b < KB; ++b) {
                    at_tma_load_2d(sK + s * K_BYTES + b * KV_BLOCK, &mapK, kv_full(s), b * 64, y);
                    at_tma_load_2d(sV + s * V_BYTES + b * KV_BLOCK, &mapV, kv_full(s), b * 64, y);
                }
                issued = it + 1;
            }
            if (*abort_flag) {
                for (int it = max(0, issued - AT_STAGES); it < issued; ++it) {
                    const long long t0 = clock64();
                    while (!at_mbar_try_wait(kv_full(it % AT_STAGES), (uint32_t)(it / AT_STAGES) & 1u) &&
                           clock64() - t0 < 20000000ll) {}
                }
            }
        }
    } else if (warp == 5) {
        if (lane == 0 && n_tiles_k > 0) {
            // S = Q K^T: M 128, N 64, both K-major. P V: M 128, N HD, A K-major, B MN-major.
            constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(AT_KEYS >> 3) << 17) |
                                         ((uint32_t)(AT_ROWS >> 4) << 24);
            constexpr uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) |
                                          ((uint32_t)(AT_ROWS >> 4) << 24);
            auto mma_s = [&](int it) {
                const int s = it % AT_STAGES;
#pragma unroll
                for (int b = 0; b < KB; ++b) {
                    const uint64_t qd = at_desc_kmajor(sQ + b * (AT_ROWS * 128));
                    const uint64_t kd = at_desc_kmajor(sK + s * K_BYTES + b * KV_BLOCK);
#pragma unroll
                    for (int k = 0; k < 4; ++k) at_mma(tmem_s, qd + (uint64_t)(k * 2), kd + (uint64_t)(k * 2), idesc_s, (b | k) ? 1u : 0u);
                }
                at_commit(s_full);
            };
            bool ok = at_mbar_wait(q_ready, 0, abort_flag) && at_mbar_wait(kv_full(0), 0, abort_flag);
            if (ok) {
                at_fence_after();
                mma_s(0);
            }
            for (int it = 0; it < n_tiles_k && ok; ++it) {
                const int s = it % AT_STAGES;
                if (it + 1 < n_tiles_k) {
                    // next page's S as soon as its keys are here and this page's S has been read
                    ok = at_mbar_wait(kv_full((it + 1) % AT_STAGES), (uint32_t)((it + 1) / AT_STAGES) & 1u, abort_flag) &&
                         at_mbar_wait(s_empty, (uint32_t)it & 1u, abort_flag);
                    if (!ok) break;
                    at_fence_after();
                    mma_s(it + 1);
                }
                ok = at_mbar_wait(p_full, (uint32_t)it & 1u, abort_flag);
                if (!ok) break;
                at_fence_after();
                const uint64_t pd = at_desc_kmajor(sP);
                const uint64_t vd = at_desc_mnmajor(sV + s * V_BYTES, KV_BLOCK);
#pragma unroll
                for (int k = 0; k < 4; ++k)        // 16 keys per MMA: 32 bytes along P's rows, 2 key groups of V
                    at_mma(tmem_pv, pd + (uint64_t)(k * 2), vd + (uint64_t)(k * 128), idesc_pv, (it | k) ? 1u : 0u);
                at_commit(pv_full);
                at_commit(kv_empty(s));
            }
        }
    } else {
        // softmax: thread i owns row i
        const int i = threadIdx.x;
        const int r_local = i / hpc;
        const int hg = chunk * hpc + (i - r_local * hpc);
        const bool valid = (r_local < rows_in_tile) && (hg < group);
        const int pos = start + q0 + r_local;
        const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
        const size_t row = (size_t)(row0 + q0 + r_local);
        const int head = kvh * group + hg;
        {   // this row of Q into the swizzled tile
            const uint4* src = reinterpret_cast<const uint4*>((const bf16*)p.q + row * p.q_stride + (size_t)head * HD);
#pragma unroll
            for (int b = 0; b < KB; ++b)
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 v = valid ? src[b * 8 + c] : make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4*>(gQ + b * (AT_ROWS * 128) + at_swizzled(i, c)) = v;
                }
            at_fence_async_smem();
            at_mbar_arrive(q_ready);
        }
        // smallest "lowest visible key" over the block's rows (first row), for the unmasked fast path
        const int blk_lo = p.window > 0 ? max(0, start + q0 + rows_in_tile - 1 - p.window + 1) : 0;
        const float sl2 = p.scale * 1.4426950408889634f;       // scores are kept raw; exp2((s - m) * scale * log2 e)
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        // m is the reference the exponentials are taken against. It follows the running maximum
        // lazily: it moves only when the maximum has grown by more than 8 powers of two, so the
        // output rows in tensor memory rarely need rescaling (the result is the same: numerator
        // and denominator share the reference).
        float m = -CUDART_INF_F, l = 0.f;
        bool ok = true;
        for (int it = 0; it < n_tiles_k && ok; ++it) {
            const int t = t_first + it;
            ok = at_mbar_wait(s_full, (uint32_t)it & 1u, abort_flag);
            if (!ok) break;
            at_fence_after();
            float s[AT_KEYS];
            at_ld32_nowait(tmem_s + lane_base, s);
            at_ld32_nowait(tmem_s + lane_base + 32, s + 32);
            at_ld_wait();
            at_fence_before();
            at_mbar_arrive(s_empty);
            float mx = -CUDART_INF_F;
            const int key0 = t * AT_KEYS;
            // A page that every row of the block sees whole needs no masking (block-uniform test).
            const bool page_whole = key0 + AT_KEYS <= start + q0 + 1 && key0 >= blk_lo;
            if (!page_whole) {
#pragma unroll
                for (int c = 0; c < AT_KEYS; ++c) {
                    const bool in = valid && key0 + c <= pos && key0 + c >= lo;
                    s[c] = in ? s[c] : -CUDART_INF_F;
                }
            }
            {   // eight independent chains of three-input maxima, not one chain of 64
                float mx8[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) mx8[j] = at_max3(s[j], s[8 + j], s[16 + j]);
#pragma unroll
                for (int c = 24; c + 16 <= AT_KEYS; c += 16)
#pragma unroll
                    for (int j = 0; j < 8; ++j) mx8[j] = at_max3(mx8[j], s[c + j], s[c + 8 + j]);
#pragma unroll
                for (int j = 0; j < 8; ++j) mx8[j] = fmaxf(mx8[j], s[56 + j]);
                mx = fmaxf(at_max3(mx8[0], mx8[1], mx8[2]), at_max3(mx8[3], mx8[4], mx8[5]));
                mx = at_max3(mx, mx8[6], mx8[7]);
            }
            float corr = 1.0f;
            if (mx > m && (m == -CUDART_INF_F || (mx - m) * sl2 > 8.0f)) {
                corr = (m == -CUDART_INF_F) ? 0.f : at_exp2((m - mx) * sl2);
                m = mx;
            }
            const float m_use = (m == -CUDART_INF_F) ? 0.f : m;
            uint32_t pk[AT_KEYS / 2];
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};       // four chains of adds, always in this order
            const float neg = -m_use * sl2;
#pragma unroll
            for (int c = 0; c < AT_KEYS; c += 2) {
                const float e0 = at_exp2(fmaf(s[c], sl2, neg)), e1 = at_exp2(fmaf(s[c + 1], sl2, neg));
                sum4[(c >> 1) & 3] += e0 + e1;
                __nv_bfloat162 h = __floats2bfloat162_rn(e0, e1);
                pk[c >> 1] = *reinterpret_cast<uint32_t*>(&h);
            }
            const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            if (it > 0) {
                // The product of the page before is complete: its P tile is free, and the output
                // rows in tensor memory can be rescaled if a row of this warp moved its reference.
                ok = at_mbar_wait(pv_full, (uint32_t)(it - 1) & 1u, abort_flag);
                if (!ok) break;
                at_fence_after();
                if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
                    for (int c = 0; c < HD; c += 32) {
                        float ov[32];
                        at_ld32_nowait(tmem_pv + lane_base + c, ov);
                        at_ld_wait();
#pragma unroll
                        for (int d = 0; d < 32; ++d) ov[d] *= corr;
                        at_st32(tmem_pv + lane_base + c, ov);
                    }
                    at_st_wait();
                }
            }
            l = l * corr + sum;
            // probabilities into the swizzled tile (the MMA that read it last has completed: pv_full)
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(gP + at_swizzled(i, c)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            if ((t + 1) * AT_KEYS > kend) {
                // value rows past the end of the sequence: zero them, whatever the page holds
                ok = at_mbar_wait(kv_full(it % AT_STAGES), (uint32_t)(it / AT_STAGES) & 1u, abort_flag);
                if (!ok) break;
                if (i < AT_KEYS && t * AT_KEYS + i >= kend) {
#pragma unroll
                    for (int b = 0; b < KB; ++b)
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            *reinterpret_cast<uint4*>(gV + (it % AT_STAGES) * V_BYTES + b * KV_BLOCK + at_swizzled(i, c)) =
                                make_uint4(0u, 0u, 0u, 0u);
                }
            }
            at_fence_async_smem();
            at_fence_before();
            at_mbar_arrive(p_full);
        }
        if (ok && n_tiles_k > 0) {
            ok = at_mbar_wait(pv_full, (uint32_t)(n_tiles_k - 1) & 1u, abort_flag);
            if (ok) {
                at_fence_after();
                const float inv = valid ? 1.0f / l : 0.f;
                bf16* dst = (bf16*)p.out + row * p.out_stride + (size_t)head * HD;
#pragma unroll
                for (int c = 0; c < HD; c += 32) {
                    float ov[32];
                    at_ld32_nowait(tmem_pv + lane_base + c, ov);
                    at_ld_wait();
                    uint32_t w[16];
#pragma unroll
                    for (int d = 0; d < 16; ++d) {
                        __nv_bfloat162 h = __floats2bfloat162_rn(ov[2 * d] * inv, ov[2 * d + 1] * inv);
                        w[d] = *reinterpret_cast<uint32_t*>(&h);
                    }
                    if (valid) {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            reinterpret_cast<uint4*>(dst + c)[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
                    }
                }
            }
        }
    }
    at_fence_before();
    __syncthreads();
    if (warp == 5) {
        at_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_s), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(ap.err, 4);
}

// ------------------------------------------------------------------------------------
typedef CUresult (*AtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static AtEncodeFn at_encode_fn() {
    static AtEncodeFn fn = nullptr;
    if (!fn) {
        void* q = nullptr;
        cudaDriverEntryPointQueryResult r;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &q, cudaEnableDefault, &r) == cudaSuccess &&
            r == cudaDriverEntryPointSuccess)
            fn = (AtEncodeFn)q;
    }
    return fn;
}
// The page pool of one layer as a matrix [pages * kv_heads * 64 rows, head_dim]: boxes of 64 x 64.
static int at_make_map(CUtensorMap* map, const void* base, long rows, int head_dim) {
    AtEncodeFn fn = at_encode_fn();
    if (!fn) return CML_ERR_BAD_SIZE;
    if ((uintptr_t)base & 15) return CML_ERR_BAD_ALIGN;
    cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
    cuuint32_t box[2] = {64, AT_KEYS};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : CML_ERR_BAD_SIZE;
}

template <int HD>
static int at_launch(const CUtensorMap& mk, const CUtensorMap& mv, AtParams ap, int n_tiles, cudaStream_t s) {
    constexpr int KB = HD / 64;
    constexpr size_t smem = 1024 + (size_t)AT_ROWS * 128 * KB + AT_ROWS * 128 + 2 * AT_STAGES * AT_KEYS * 128 * KB + 256;
    if ((long)n_tiles * ap.a.n_kv_heads * ap.a.head_chunks > 0x7fffffffL) return CML_ERR_BAD_SIZE;
    ap.n_tiles = n_tiles;
    dim3 grid((unsigned)(n_tiles * ap.a.n_kv_heads * ap.a.head_chunks), 1, 1);
    cudaError_t e = cml_allow_smem<attn_prefill_tc_kernel<HD>>(smem);
    if (e != cudaSuccess) return (int)e;
    e = launch_pdl(attn_prefill_tc_kernel<HD>, grid, dim3(AT_THREADS), smem, s, mk, mv, ap);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// Tiles of rows_per_tile tokens with rows_per_tile * heads_per_cta <= 128; n_pages: pages of the pool.
// q rows must be 16-byte aligned (q_stride and head_dim multiples of 8), the output likewise.
extern "C" int cml_attn_prefill_tc(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                   const void* v_pages, long n_pages, const int* block_table, int max_blocks,
                                   const int* tile_seq, const int* tile_q0, int n_tiles, const int* seq_row0,
                                   const int* seq_start, const int* seq_new, int n_heads, int n_kv_heads, int head_dim,
                                   int rows_per_tile, int heads_per_cta, int head_chunks, int window, float scale,
                                   int* err, void* stream) {
    if (n_tiles <= 0) return 0;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return CML_ERR_BAD_SIZE;
    if (rows_per_tile < 1 || heads_per_cta < 1 || rows_per_tile * heads_per_cta > AT_ROWS) return CML_ERR_BAD_SIZE;
    if (heads_per_cta * head_chunks < n_heads / n_kv_heads) return CML_ERR_BAD_SIZE;
    if ((q_stride & 7) || (out_stride & 7) || ((uintptr_t)q & 15) || ((uintptr_t)out & 15)) return CML_ERR_BAD_ALIGN;
    if (head_dim != 64 && head_dim != 128) return CML_ERR_BAD_SIZE;
    CUtensorMap mk, mv;
    const long rows = n_pages * n_kv_heads * CML_PAGE;
    int rc = at_make_map(&mk, k_pages, rows, head_dim);
    if (rc) return rc;
    rc = at_make_map(&mv, v_pages, rows, head_dim);
    if (rc) return rc;
    AtParams ap;
    AttnParams& p = ap.a;
    p.q = q; p.q_stride = q_stride; p.out = out; p.out_stride = out_stride;
    p.k_pages = k_pages; p.v_pages = v_pages; p.block_table = block_table; p.max_blocks = max_blocks;
    p.tile_seq = tile_seq; p.tile_q0 = tile_q0; p.seq_row0 = seq_row0; p.seq_start = seq_start; p.seq_new = seq_new;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim;
    p.rows_per_tile = rows_per_tile; p.heads_per_cta = heads_per_cta; p.head_chunks = head_chunks;
    p.n_splits = 1; p.window = window; p.scale = scale; p.partial = nullptr; p.tickets = nullptr;
    ap.err = err;
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 64) return at_launch<64>(mk, mv, ap, n_tiles, s);
    return at_launch<128>(mk, mv, ap, n_tiles, s);
}
