// bfloat16 matrix products on the fifth-generation tensor cores: TMA loads into swizzled
// shared memory, tcgen05.mma issued by one thread with the accumulator in tensor memory,
// tcgen05.ld in the epilogue. One kernel serves decode and prefill steps of few rows; steps
// of many rows run its two-block form (gemm_tc_pair_kernel, tcgen05 cta_group::2) below:
//
//   D[128 x BN] tile = Arows[128, K] * Brows[BN, K]^T        (both operands K-major)
//
// * prefill of up to 128 rows: Arows = activations [tokens, K], Brows = weights [out, K];
//   BN = 128 or 256; epilogues: store bfloat16, store float, add into the float residual
//   stream, SwiGLU on packed gate/up rows (interleaved in groups of 16 output columns).
// * decode ("transposed"): Arows = weights [out, K], Brows = activations [batch, K] with
//   BN = 16..64 >= batch, so every weight byte crosses the memory bus once and no tensor-core
//   row is wasted on padding; K may be split (the split is part of the work item's number),
//   each split writing a float partial [split][batch][out] that the consumer sums in order
//   (no atomics: the result does not depend on timing); epilogues: float partial, SwiGLU to
//   bfloat16 (no split). The output head, with many times more tiles than SMs, runs on
//   persistent blocks.
//
// It stands where the reference runs q8_gemv / q8_gemm_batched
// (src/cuda_resident.rs:230, :1494), whose batched form re-reads the weights once per 8
// tokens (src/cuda_resident.rs:8824-8847).
//
// Warp roles (192 threads): warp 0 lane 0 issues TMA loads through a ring of stages, warp 1
// allocates tensor memory and lane 0 issues the MMAs, warps 2-5 read the accumulator (each
// its own quarter of the 128 lanes) and write the result. Every wait on an mbarrier is
// bounded: when a bound is hit the kernel sets *err, lets its copies land, frees its tensor
// memory and returns. No load uses cluster multicast.
#include "common.cuh"
#include <cuda.h>

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define TC_WAIT_CYCLES 2000000000ll

enum { TC_STORE = 0, TC_STORE_F32 = 1, TC_ADD_F32 = 2, TC_SWIGLU = 3, TC_T_PARTIAL = 4, TC_T_SWIGLU = 5, TC_ADD_NORM = 6 };

struct TcParams {
    void* C;            // output (type by epilogue)
    long ldc;           // row stride of C in elements
    int rowsA, rowsB;   // valid rows of the two operands
    int num_kb;         // k-blocks of 64 in total
    int kb_per_split;
    int tiles_a, tiles_b, splits;   // work items
    int independent;    // operand that no earlier kernel writes (weights): 0 = A, 1 = B
    int* err;
    // Two-block kernel only. A norm between two products is split over them: the product before
    // it (TC_ADD_NORM) adds into the residual stream C, writes x_out = bfloat16(C * norm_w) and
    // the sum of squares of its 256 columns of every row; the product after it reads rows of
    // x_out and multiplies its own output rows by rsqrt(sum of those sums / in_hidden + in_eps),
    // which is what the norm's scale would have done to its input rows.
    const void* norm_w; // [rowsB] weight of the norm after this product
    int norm_w_dtype;
    bf16* x_out;        // [rowsA, rowsB] (row stride ldx)
    long ldx;
    float* out_sumsq;   // [tiles_b][rowsA]
    const float* in_sumsq;  // [in_parts][rowsA], or null: the rows of A are complete
    int in_parts;
    float in_inv_hidden, in_eps;
    int staged_ok;      // the outputs are aligned for 16-byte (float) and 8-byte (bfloat16) row pieces
    long split_stride;  // TC_STORE_F32 of a product split over K: split s writes C + s * split_stride (elements)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false (and *abort set) when the bound is hit or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > TC_WAIT_CYCLES) {
            *abort_flag = 1;
            return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
// The first copy through a tensor map fetches the map itself: asked for at kernel entry, that
// round trip runs beside the set-up instead of before the first tile.
__device__ __forceinline__ void tc_prefetch_map(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)map) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tc_ld16_nowait(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bfloat16),
// 128-byte swizzled as TMA writes it: start address, leading offset 1 (unused for swizzled
// K-major), stride 1024 bytes between groups of 8 rows, version 1, layout SWIZZLE_128B.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Stages of the ring. Decode tiles (bn <= 64) with little work per block keep a small ring so
// that several blocks fit an SM: the blocks of the next kernel then become resident while
// this one still runs and prefetch their weights. Blocks that stream many k-blocks take a
// deeper ring, but for tiles of 16 batch rows only 5 stages (90 KB, two blocks an SM): what is
// in flight matters less there than the next product's blocks starting early; tiles of 32 and
// 64 batch rows were slower with fewer stages than these. (The figures are in profiles/README.md.)
__host__ __device__ constexpr int tc_stages(int bn, bool deep) {
    return bn >= 256 ? 4 : (bn >= 128 ? 6 : (deep ? (bn >= 64 ? 8 : (bn >= 32 ? 10 : 5)) : 4));
}
__host__ __device__ constexpr int tc_tmem_cols(int bn) { return bn <= 16 ? 32 : (bn <= 32 ? 64 : (bn <= 64 ? 128 : (bn <= 128 ? 256 : 512))); }
__host__ __device__ constexpr size_t tc_smem_bytes(int bn, bool deep) {
    return 1024 /*alignment slack*/ + (size_t)tc_stages(bn, deep) * (TC_BM * 128 + bn * 128) + 512 /*barriers*/;
}

// rsqrt(sum_t sumsq[t][row] / hidden + eps): the scale a row still lacks when the norm before a
// product was split over the products around it. The sums are added in index order; every
// load is unconditional (of a clamped place) so that all are in flight together.
__device__ __forceinline__ float tc_row_scale(const float* __restrict__ sumsq, int parts, int rows, int row,
                                              float inv_hidden, float eps) {
    float ssq = 0.f;
    for (int t0 = 0; t0 < parts; t0 += 16) {
        float t[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) t[i] = sumsq[(size_t)min(t0 + i, parts - 1) * rows + row];
#pragma unroll
        for (int i = 0; i < 16; ++i) ssq += (t0 + i < parts) ? t[i] : 0.f;
    }
    return 1.0f / sqrtf(ssq * inv_hidden + eps);
}

// One 16-column chunk of one accumulator row, already in registers, to its place in the output.
template <int EPI>
__device__ __forceinline__ void tc_epilogue_chunk(const TcParams& p, const uint32_t (&r)[16], const uint32_t (&u)[16],
                                                  int rowA, int colB, int split, int lane, int a_group0) {
    if (EPI == TC_STORE || EPI == TC_STORE_F32 || EPI == TC_ADD_F32) {
        if (rowA >= p.rowsA || colB >= p.rowsB) return;
        const int n_ok = min(16, p.rowsB - colB);
        if (EPI == TC_STORE) {
            bf16* dst = (bf16*)p.C + (size_t)rowA * p.ldc + colB;
            if (n_ok == 16 && (((uintptr_t)dst & 15) == 0)) {
                uint32_t w[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                    w[i] = *reinterpret_cast<uint32_t*>(&h);
                }
                reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
            } else {
                for (int i = 0; i < n_ok; ++i) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
            }
        } else {
            float* dst = (float*)p.C + (size_t)split * p.split_stride + (size_t)rowA * p.ldc + colB;
            if (n_ok == 16 && (((uintptr_t)dst & 15) == 0)) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float4 v = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                           __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
                    if (EPI == TC_ADD_F32) {
                        const float4 o = reinterpret_cast<float4*>(dst)[i];
                        v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                    }
                    reinterpret_cast<float4*>(dst)[i] = v;
                }
            } else {
                for (int i = 0; i < n_ok; ++i) {
                    const float v = __uint_as_float(r[i]);
                    dst[i] = (EPI == TC_ADD_F32) ? dst[i] + v : v;
                }
            }
        }
    } else if (EPI == TC_SWIGLU) {
        // r: 16 gate columns, u: the 16 up columns of the same outputs
        const int out_col = colB / 2;
        const int inter = p.rowsB / 2;
        if (rowA >= p.rowsA || out_col >= inter) return;
        bf16* dst = (bf16*)p.C + (size_t)rowA * p.ldc + out_col;
        const int n_ok = min(16, inter - out_col);
        float a[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float g = __uint_as_float(r[i]);
            a[i] = __fdividef(g, 1.0f + __expf(-g)) * __uint_as_float(u[i]);
        }
        if (n_ok == 16 && (((uintptr_t)dst & 15) == 0)) {
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                __nv_bfloat162 h = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
                w[i] = *reinterpret_cast<uint32_t*>(&h);
            }
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
        } else {
            for (int i = 0; i < n_ok; ++i) dst[i] = __float2bfloat16_rn(a[i]);
        }
    } else if (EPI == TC_T_PARTIAL) {
        // transposed: this thread owns output feature rowA for 16 batch rows
        if (rowA >= p.rowsA) return;
        float* dst = (float*)p.C + ((size_t)split * p.rowsB) * p.ldc + rowA;
        const int n_ok = min(16, p.rowsB - colB);
        for (int i = 0; i < n_ok; ++i) dst[(size_t)(colB + i) * p.ldc] = __uint_as_float(r[i]);
    } else {   // TC_T_SWIGLU: lanes 0-15 hold gate rows, lanes 16-31 the up rows of the same outputs
        const int inter = p.rowsA / 2;
        const int out_j = a_group0 / 2 + (lane & 15);
        const int n_ok = min(16, p.rowsB - colB);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float mine = __uint_as_float(r[i]);
            const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
            if (lane < 16 && i < n_ok && out_j < inter)
                ((bf16*)p.C)[(size_t)(colB + i) * p.ldc + out_j] =
                    __float2bfloat16_rn(__fdividef(mine, 1.0f + __expf(-mine)) * other);
        }
    }
}

// Work items are (tile of A rows, tile of B rows, split of K), numbered with the A tile
// fastest; a block takes items blockIdx.x, blockIdx.x + gridDim.x, ... The accumulator is
// double-buffered in tensor memory, so while the epilogue warps drain one item the MMA
// thread already runs the next one.
template <int BN, int EPI, bool DEEP>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, TcParams p) {
    constexpr int STAGES = tc_stages(BN, DEEP);
    constexpr uint32_t A_BYTES = TC_BM * 128, B_BYTES = BN * 128;
    constexpr uint32_t TMEM_COLS = tc_tmem_cols(BN);          // two accumulators of BN columns
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t smemA = base, smemB = base + STAGES * A_BYTES;
    const uint32_t bars = smemB + STAGES * B_BYTES;   // full[S], empty[S], acc_full[2], acc_empty[2]; tmem slot; abort
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + STAGES * (A_BYTES + B_BYTES) + (2 * STAGES + 4) * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full = [&](int b) { return bars + 8u * (2 * STAGES + b); };
    auto acc_empty = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_work = p.tiles_a * p.tiles_b * p.splits;
    if (threadIdx.x == 32) {
        tc_prefetch_map(&mapA);
        tc_prefetch_map(&mapB);
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 128);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    auto item = [&](int w, int& a0, int& b0, int& split, int& kb_begin, int& n_kb) {
        const int ta = w % p.tiles_a;
        const int rest = w / p.tiles_a;
        const int tb = rest % p.tiles_b;
        split = rest / p.tiles_b;
        a0 = ta * TC_BM;
        b0 = tb * BN;
        kb_begin = split * p.kb_per_split;
        n_kb = max(0, min(p.num_kb, kb_begin + p.kb_per_split) - kb_begin);
    };

    if (warp == 0) {
        if (lane == 0) {
            int g = 0;                      // k-blocks issued so far by this block, over all its items
            bool waited = false, ok = true;
            for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
                int a0, b0, split, kb_begin, n_kb;
                item(w, a0, b0, split, kb_begin, n_kb);
                int i = 0;
                if (!waited) {
                    // The weights do not depend on the kernel before: their first tiles are on
                    // their way before this kernel waits for that kernel's results.
                    const int pre = min(n_kb, STAGES);
                    for (; i < pre; ++i) {
                        mbar_expect_tx(full_bar(i), A_BYTES + B_BYTES);
                        const int k = (kb_begin + i) * TC_BK;
                        if (p.independent == 0) tma_load_2d(smemA + i * A_BYTES, &mapA, full_bar(i), k, a0);
                        else tma_load_2d(smemB + i * B_BYTES, &mapB, full_bar(i), k, b0);
                    }
                    pdl_wait();
                    waited = true;
                    for (int j = 0; j < pre; ++j) {
                        const int k = (kb_begin + j) * TC_BK;
                        if (p.independent == 0) tma_load_2d(smemB + j * B_BYTES, &mapB, full_bar(j), k, b0);
                        else tma_load_2d(smemA + j * A_BYTES, &mapA, full_bar(j), k, a0);
                    }
                    g = pre;
                }
                for (; i < n_kb; ++i, ++g) {
                    const int s = g % STAGES;
                    const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(full_bar(s), A_BYTES + B_BYTES);
                    const int k = (kb_begin + i) * TC_BK;
                    tma_load_2d(smemA + s * A_BYTES, &mapA, full_bar(s), k, a0);
                    tma_load_2d(smemB + s * B_BYTES, &mapB, full_bar(s), k, b0);
                }
            }
            if (*abort_flag) {
                // let the copies that are in flight land before the block leaves
                for (int i = max(0, g - STAGES); i < g; ++i) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(full_bar(i % STAGES), (uint32_t)(i / STAGES) & 1u) &&
                           clock64() - t0 < 20000000ll) {}
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                       ((uint32_t)(TC_BM >> 4) << 24);
            int g = 0, j = 0;                             // j counts the items that have k-blocks
            bool ok = true;
            for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
                int a0, b0, split, kb_begin, n_kb;
                item(w, a0, b0, split, kb_begin, n_kb);
                if (n_kb == 0) continue;                  // the epilogue writes zeros on its own
                const int buf = j & 1;
                // the epilogue must have drained this accumulator (two items ago)
                ok = mbar_wait(acc_empty(buf), (((uint32_t)j >> 1) & 1u) ^ 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                for (int i = 0; i < n_kb && ok; ++i, ++g) {
                    const int s = g % STAGES;
                    const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
                    ok = mbar_wait(full_bar(s), ph, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t adesc = smem_desc_sw128(smemA + s * A_BYTES);
                    const uint64_t bdesc = smem_desc_sw128(smemB + s * B_BYTES);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        tc_mma_bf16(tmem_d, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (i | k) ? 1u : 0u);
                    tc_commit(empty_bar(s));         // the stage is free once these MMAs have read it
                }
                if (ok) tc_commit(acc_full(buf));    // the accumulator is complete
                ++j;
            }
        }
    } else {
        const int q = warp & 3;                  // the quarter of tensor-memory lanes this warp may read
        pdl_wait();                              // the output may still be read by a kernel before
        bool ok = true;
        int j = 0;                               // counts the items that have k-blocks, as the MMA thread does
        for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
            int a0, b0, split, kb_begin, n_kb;
            item(w, a0, b0, split, kb_begin, n_kb);
            const int buf = j & 1;
            const int rowA = a0 + q * 32 + lane;
            if (n_kb > 0) {
                ok = mbar_wait(acc_full(buf), ((uint32_t)j >> 1) & 1u, abort_flag);
                if (!ok) break;
            }
            tc_fence_after();
            const uint32_t taddr = tmem_base + (uint32_t)(buf * BN) + ((uint32_t)(q * 32) << 16);
            constexpr int STEP = (EPI == TC_SWIGLU) ? 32 : 16;
#pragma unroll 1
            for (int c = 0; c < BN; c += STEP) {
                uint32_t r[16], u[16];
                if (n_kb > 0) {
                    tc_ld16(taddr + c, r);
                    if (EPI == TC_SWIGLU) tc_ld16(taddr + c + 16, u);
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) r[i] = 0u, u[i] = 0u;
                }
                tc_epilogue_chunk<EPI>(p, r, u, rowA, b0 + c, split, lane, a0 + q * 32);
            }
            if (n_kb > 0) {
                tc_fence_before();
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty(buf)) : "memory");
                ++j;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.err, 2);
}

// TC_ADD_NORM, 16 columns of one row: C += accumulator; x_out = bfloat16(C * norm_w); returns the
// sum of squares of the new C values (zero for columns beyond the matrix).
__device__ __forceinline__ float tc_add_norm_chunk(const TcParams& p, const uint32_t (&r)[16], int rowA, int colB) {
    if (rowA >= p.rowsA || colB >= p.rowsB) return 0.f;
    const int n_ok = min(16, p.rowsB - colB);
    float* dst = (float*)p.C + (size_t)rowA * p.ldc + colB;
    bf16* xo = p.x_out + (size_t)rowA * p.ldx + colB;
    float v[16], g[16];
    const bool vec = n_ok == 16 && (((uintptr_t)dst & 15) == 0) && (((uintptr_t)xo & 15) == 0);
    if (vec) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 o = reinterpret_cast<const float4*>(dst)[i];
            v[4 * i] = o.x; v[4 * i + 1] = o.y; v[4 * i + 2] = o.z; v[4 * i + 3] = o.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = i < n_ok ? dst[i] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int col = colB + min(i, n_ok - 1);
        g[i] = p.norm_w_dtype == CML_DTYPE_F32 ? ((const float*)p.norm_w)[col] : __bfloat162float(((const bf16*)p.norm_w)[col]);
    }
    float ssq = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        v[i] = i < n_ok ? v[i] + __uint_as_float(r[i]) : 0.f;
        ssq = fmaf(v[i], v[i], ssq);
    }
    if (vec) {
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i] * g[2 * i], v[2 * i + 1] * g[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        reinterpret_cast<uint4*>(xo)[0] = make_uint4(w[0], w[1], w[2], w[3]);
        reinterpret_cast<uint4*>(xo)[1] = make_uint4(w[4], w[5], w[6], w[7]);
    } else {
        for (int i = 0; i < n_ok; ++i) {
            dst[i] = v[i];
            xo[i] = __float2bfloat16_rn(v[i] * g[i]);
        }
    }
    return ssq;
}

// ------------------------------------------------------------------------------------
// Two blocks of a cluster on one tile (tcgen05 cta_group::2): D[256 x 256] = Arows[256, K] *
// Brows[256, K]^T. Each block of the pair loads its own 128 rows of A and its own 128 rows of B
// (16 KB + 16 KB a stage instead of 16 KB + 32 KB for a 128 x 256 tile of one block), the
// leader's MMA thread issues 256 x 256 x 16 MMAs for both, and each block ends up with its 128
// rows of the tile in its own tensor memory. A third less shared-memory and L2 traffic per
// flop than the one-block tile, which is what bounds large products.
//
// Barriers live at the same offsets in both blocks. full[s] is used in the leader only: its
// producer expects the bytes of both blocks, and both blocks' TMA loads report to it
// (cp.async.bulk.tensor with .cta_group::2 and no multicast). empty[s] and acc_full[b] are
// signalled in both blocks at once by the leader's tcgen05.commit with .multicast::cluster;
// acc_empty[b] is the leader's, and the epilogue warps of both blocks arrive on it.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
    return r;
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"((uint64_t)map), "r"(leader_bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3)
                 : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}

#define TC_PAIR_STAGES 6
#define TC_STAGE_LD 36       // floats between rows of an epilogue warp's staging tile (conflict-free 16-byte accesses)
__host__ __device__ constexpr size_t tc_pair_smem_bytes() {
    return 1024 + (size_t)TC_PAIR_STAGES * (2 * TC_BM * 128) + 512 + 4 * 32 * TC_STAGE_LD * sizeof(float);
}

// Work items are tiles of 256 A rows by 256 B rows, A tile fastest; cluster c takes items
// c, c + clusters, ... p.tiles_a and p.tiles_b count those tiles. No split of K.
template <int EPI, int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, TcParams p) {
    constexpr int STAGES = TC_PAIR_STAGES;
    constexpr uint32_t A_BYTES = TC_BM * 128, B_BYTES = (BN / 2) * 128;   // this block's halves of a stage
    constexpr uint32_t TMEM_COLS = 512;                                    // two accumulators of BN columns; all of the SM's
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t smemA = base, smemB = base + STAGES * A_BYTES;
    const uint32_t bars = smemB + STAGES * B_BYTES;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + STAGES * (A_BYTES + B_BYTES) + (2 * STAGES + 4) * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* stage = reinterpret_cast<float*>(gen_base + STAGES * (A_BYTES + B_BYTES) + 512);   // [4 warps][32][TC_STAGE_LD]
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full = [&](int b) { return bars + 8u * (2 * STAGES + b); };
    auto acc_empty = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 32) {
        tc_prefetch_map(&mapA);
        tc_prefetch_map(&mapB);
    }
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int cluster = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const int n_tiles = p.tiles_a * p.tiles_b;
    const int n_work = n_tiles * p.splits;       // a split of K is a work item of its own (float partial sums)

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 8);          // one lane of each epilogue warp of both blocks
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        // All 512 columns: the allocation only returns once the SM's tensor memory is free of
        // other blocks, so both blocks of the pair get the same base (the MMA addresses both).
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) {
        uint32_t other;
        asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(other) : "r"(map_to_cta(smem_u32(tmem_slot), rank ^ 1u)));
        if (other != tmem_base) *abort_flag = 1;         // both blocks see the mismatch and give up
    }
    __syncthreads();
    pdl_launch_dependents();

    // Items are numbered so that the clusters at work at one time share operands that fit L2:
    // the tiles of A in groups of 8, all tiles of B for a group before the next group. (With
    // the A tile simply fastest, a product of 16,384 rows streamed all of A from HBM once per
    // tile of B.)
    auto item = [&](int w, int& a0, int& b0) {
        w %= n_tiles;                                    // splits of K are the slowest index
        constexpr int G = 8;
        const int per_group = G * p.tiles_b;
        const int g = w / per_group, within = w - g * per_group;
        const int gsz = min(G, p.tiles_a - g * G);
        const int tb = within / gsz, ta = g * G + (within - tb * gsz);
        a0 = ta * 256 + (int)rank * TC_BM;
        b0 = tb * BN + (int)rank * (BN / 2);
    };
    auto k_range = [&](int w, int& kb0) {                // first k-block and number of k-blocks of item w
        kb0 = (w / n_tiles) * p.kb_per_split;
        return min(p.kb_per_split, p.num_kb - kb0);
    };

    if (warp == 0) {
        if (lane == 0 && !*abort_flag) {
            int g = 0;
            bool waited = false, ok = true;
            auto leader_full = [&](int s) { return map_to_cta(full_bar(s), 0); };
            for (int w = cluster; w < n_work && ok; w += n_clusters) {
                int a0, b0, kb0;
                item(w, a0, b0);
                const int nkb = k_range(w, kb0);
                int i = 0;
                if (!waited) {
                    const int pre = min(nkb, STAGES);
                    for (; i < pre; ++i) {
                        if (leader) mbar_expect_tx(full_bar(i), 2 * (A_BYTES + B_BYTES));
                        if (p.independent == 0) tma_load_2d_pair(smemA + i * A_BYTES, &mapA, leader_full(i), (kb0 + i) * TC_BK, a0);
                        else tma_load_2d_pair(smemB + i * B_BYTES, &mapB, leader_full(i), (kb0 + i) * TC_BK, b0);
                    }
                    pdl_wait();
                    waited = true;
                    for (int j = 0; j < pre; ++j) {
                        if (p.independent == 0) tma_load_2d_pair(smemB + j * B_BYTES, &mapB, leader_full(j), (kb0 + j) * TC_BK, b0);
                        else tma_load_2d_pair(smemA + j * A_BYTES, &mapA, leader_full(j), (kb0 + j) * TC_BK, a0);
                    }
                    g = pre;
                }
                for (; i < nkb; ++i, ++g) {
                    const int s = g % STAGES;
                    const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
                    if (leader) mbar_expect_tx(full_bar(s), 2 * (A_BYTES + B_BYTES));
                    tma_load_2d_pair(smemA + s * A_BYTES, &mapA, leader_full(s), (kb0 + i) * TC_BK, a0);
                    tma_load_2d_pair(smemB + s * B_BYTES, &mapB, leader_full(s), (kb0 + i) * TC_BK, b0);
                }
            }
            if (*abort_flag) {
                // let the copies in flight land before the block leaves (the leader sees them on
                // its barriers; the other block has none of its own and just gives them time)
                const long long t0 = clock64();
                if (leader) {
                    for (int i = max(0, g - STAGES); i < g; ++i)
                        while (!mbar_try_wait(full_bar(i % STAGES), (uint32_t)(i / STAGES) & 1u) &&
                               clock64() - t0 < 20000000ll) {}
                } else {
                    while (clock64() - t0 < 20000000ll) {}
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader && !*abort_flag) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                       ((uint32_t)(256 >> 4) << 24);
            int g = 0, j = 0;
            bool ok = true;
            for (int w = cluster; w < n_work && ok; w += n_clusters, ++j) {
                const int buf = j & 1;
                ok = mbar_wait(acc_empty(buf), (((uint32_t)j >> 1) & 1u) ^ 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * 256);
                int kb0;
                const int nkb = k_range(w, kb0);
                for (int i = 0; i < nkb && ok; ++i, ++g) {
                    const int s = g % STAGES;
                    const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
                    ok = mbar_wait(full_bar(s), ph, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t adesc = smem_desc_sw128(smemA + s * A_BYTES);
                    const uint64_t bdesc = smem_desc_sw128(smemB + s * B_BYTES);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        tc_mma_bf16_pair(tmem_d, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (i | k) ? 1u : 0u);
                    tc_commit_pair(empty_bar(s));        // frees the stage in both blocks
                }
                if (ok) tc_commit_pair(acc_full(buf));   // both blocks' halves of the tile are complete
            }
        }
    } else {
        const int q = warp & 3;
        pdl_wait();
        bool ok = !*abort_flag;
        int j = 0;
        for (int w = cluster; w < n_work && ok; w += n_clusters, ++j) {
            int a0, b0;
            item(w, a0, b0);
            b0 -= (int)rank * (BN / 2);                  // every block holds all BN columns of its rows
            const int split = w / n_tiles;
            const int buf = j & 1;
            const int rowA = a0 + q * 32 + lane;
            ok = mbar_wait(acc_full(buf), ((uint32_t)j >> 1) & 1u, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + (uint32_t)(buf * 256) + ((uint32_t)(q * 32) << 16);
            float row_scale = 1.f;                   // what the norm before this product left to it
            if (p.in_sumsq != nullptr)
                row_scale = tc_row_scale(p.in_sumsq, p.in_parts, p.rowsA, min(rowA, p.rowsA - 1), p.in_inv_hidden, p.in_eps);
            float ssq_out = 0.f;                     // sum of squares of this thread's row (columns that took the plain path)
            float ssq_st[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};   // and of rows it * 4 + lane / 8, this lane's 4 columns (staged path)
            constexpr bool CAN_STAGE = EPI == TC_STORE || EPI == TC_STORE_F32 || EPI == TC_ADD_F32 || EPI == TC_ADD_NORM;
            constexpr bool READS_C = EPI == TC_ADD_F32 || EPI == TC_ADD_NORM;
            float* st = stage + q * 32 * TC_STAGE_LD;
            const int cl = (lane & 7) * 4;           // staged path: this lane's 4 columns of a chunk ...
            const int row_base = a0 + q * 32 + (lane >> 3);   // ... of rows row_base + 4 * it
            auto staged = [&](int c) { return CAN_STAGE && p.staged_ok && c < BN && b0 + c + 32 <= p.rowsB; };
            // The loop is software-pipelined: while a chunk of 32 columns is worked on, the next
            // chunk's accumulators are on their way from tensor memory and its values of C (and
            // the norm's weight) from global memory. Either round trip, taken per chunk, was most
            // of an epilogue that took as long as the products of a 2,048-deep tile.
            auto fetch_c = [&](int c, float4 (&o)[8], float (&g4)[4]) {
                if (!READS_C || !staged(c)) return;
                const int col = b0 + c + cl;
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int grow = min(row_base + it * 4, p.rowsA - 1);          // a valid place always
                    o[it] = *reinterpret_cast<const float4*>((const float*)p.C + (size_t)grow * p.ldc + col);
                }
                if (EPI == TC_ADD_NORM) {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        g4[i] = p.norm_w_dtype == CML_DTYPE_F32 ? ((const float*)p.norm_w)[col + i]
                                                                : __bfloat162float(((const bf16*)p.norm_w)[col + i]);
                }
            };
            uint32_t r[16], u[16], rn[16], un[16];
            float4 o[8], on[8];
            float g4[4] = {1.f, 1.f, 1.f, 1.f}, g4n[4] = {1.f, 1.f, 1.f, 1.f};
            tc_ld16_nowait(taddr, rn);
            tc_ld16_nowait(taddr + 16, un);
            fetch_c(0, on, g4n);
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 16; ++i) r[i] = rn[i], u[i] = un[i];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = on[i];
#pragma unroll
                for (int i = 0; i < 4; ++i) g4[i] = g4n[i];
                if (c + 32 < BN) {
                    tc_ld16_nowait(taddr + c + 32, rn);
                    tc_ld16_nowait(taddr + c + 48, un);
                    fetch_c(c + 32, on, g4n);
                }
                if (p.in_sumsq != nullptr) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        r[i] = __float_as_uint(__uint_as_float(r[i]) * row_scale);
                        u[i] = __float_as_uint(__uint_as_float(u[i]) * row_scale);
                    }
                }
                if (staged(c)) {
                    // Through shared memory, so that a warp's accesses to the output are whole
                    // 128-byte pieces of four rows instead of 16 bytes of each of 32 rows.
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        *reinterpret_cast<uint4*>(st + lane * TC_STAGE_LD + 4 * i) = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
                        *reinterpret_cast<uint4*>(st + lane * TC_STAGE_LD + 16 + 4 * i) = make_uint4(u[4 * i], u[4 * i + 1], u[4 * i + 2], u[4 * i + 3]);
                    }
                    __syncwarp();
                    const int col = b0 + c + cl;
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int grow = row_base + it * 4;
                        float4 v = *reinterpret_cast<const float4*>(st + ((lane >> 3) + it * 4) * TC_STAGE_LD + cl);
                        if (grow >= p.rowsA) continue;
                        if (EPI == TC_STORE) {
                            __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                            *reinterpret_cast<uint2*>((bf16*)p.C + (size_t)grow * p.ldc + col) =
                                make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
                        } else {
                            if (READS_C) { v.x += o[it].x; v.y += o[it].y; v.z += o[it].z; v.w += o[it].w; }
                            *reinterpret_cast<float4*>((float*)p.C + (size_t)split * p.split_stride + (size_t)grow * p.ldc + col) = v;
                            if (EPI == TC_ADD_NORM) {
                                ssq_st[it] = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ssq_st[it]))));
                                __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * g4[0], v.y * g4[1]);
                                __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * g4[2], v.w * g4[3]);
                                *reinterpret_cast<uint2*>(p.x_out + (size_t)grow * p.ldx + col) =
                                    make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
                            }
                        }
                    }
                    __syncwarp();
                } else if (EPI == TC_SWIGLU) {
                    tc_epilogue_chunk<EPI>(p, r, u, rowA, b0 + c, 0, lane, 0);
                } else if (EPI == TC_ADD_NORM) {
                    ssq_out += tc_add_norm_chunk(p, r, rowA, b0 + c);
                    ssq_out += tc_add_norm_chunk(p, u, rowA, b0 + c + 16);
                } else {
                    tc_epilogue_chunk<EPI>(p, r, r, rowA, b0 + c, split, lane, 0);
                    tc_epilogue_chunk<EPI>(p, u, u, rowA, b0 + c + 16, split, lane, 0);
                }
            }
            if (EPI == TC_ADD_NORM) {
                // the staged sums: over the 8 lanes that share a row, then to the lane that owns the row
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    float t = ssq_st[it];
                    t += __shfl_xor_sync(0xffffffffu, t, 1);
                    t += __shfl_xor_sync(0xffffffffu, t, 2);
                    t += __shfl_xor_sync(0xffffffffu, t, 4);
                    t = __shfl_sync(0xffffffffu, t, (lane & 3) * 8);
                    if ((lane >> 2) == it) ssq_out += t;
                }
                if (rowA < p.rowsA) p.out_sumsq[(size_t)(b0 / BN) * p.rowsA + rowA] = ssq_out;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(map_to_cta(acc_empty(buf), 0)) : "memory");
        }
    }
    tc_fence_before();
    cluster_sync_all();          // no block leaves while its partner may still signal its barriers
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.err, 2);
}

// ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// A 2-D map over a row-major bfloat16 matrix [rows, K] with row stride ld (elements):
// boxes of 64 columns (128 bytes, swizzled) by box_rows rows; out-of-range parts read zero.
static int make_map(CUtensorMap* map, const void* base, long rows, long K, long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return CML_ERR_BAD_SIZE;
    if (((uintptr_t)base & 15) || ((ld * 2) & 15)) return CML_ERR_BAD_ALIGN;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : CML_ERR_BAD_SIZE;
}

template <int BN, int EPI, bool DEEP>
static int launch_tc2(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, dim3 grid, cudaStream_t s) {
    const size_t smem = tc_smem_bytes(BN, DEEP);
    cudaError_t e = cml_allow_smem<gemm_tc_kernel<BN, EPI, DEEP>>(smem);
    if (e != cudaSuccess) return (int)e;
    e = launch_pdl(gemm_tc_kernel<BN, EPI, DEEP>, grid, dim3(TC_THREADS), smem, s, ma, mb, p);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

template <int BN, int EPI>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, dim3 grid, cudaStream_t s) {
    if constexpr (BN <= 64) {
        if (p.kb_per_split >= 12) return launch_tc2<BN, EPI, true>(ma, mb, p, grid, s);
    }
    return launch_tc2<BN, EPI, false>(ma, mb, p, grid, s);
}

// A: [rowsA, K] bfloat16 (ld lda), B: [rowsB, K] bfloat16 (ld ldb).
// Normal epilogues (0..3) write C[rowA][rowB]; transposed ones (4, 5) write C[..][rowA] per rowB.
// bn: tile over B rows (64, 128 or 256; transposed: 16, 32, 64 or 128). splits > 1 only with TC_T_PARTIAL.
extern "C" int cml_gemm_tc(const void* A, long lda, int rowsA, const void* B, long ldb, int rowsB, int K, void* C,
                           long ldc, int epilogue, int bn, int splits, int* err, void* stream) {
    if (rowsA <= 0 || rowsB <= 0) return 0;
    if (K <= 0 || (K & 7)) return CML_ERR_BAD_SIZE;
    if (splits < 1 || (splits > 1 && epilogue != TC_T_PARTIAL)) return CML_ERR_BAD_SIZE;
    CUtensorMap ma, mb;
    int rc = make_map(&ma, A, rowsA, K, lda, TC_BM);
    if (rc) return rc;
    rc = make_map(&mb, B, rowsB, K, ldb, bn);
    if (rc) return rc;
    TcParams p;
    p.C = C; p.ldc = ldc; p.rowsA = rowsA; p.rowsB = rowsB;
    p.num_kb = (K + TC_BK - 1) / TC_BK;
    if (splits > p.num_kb) splits = p.num_kb;
    p.kb_per_split = (p.num_kb + splits - 1) / splits;
    p.err = err;
    p.norm_w = nullptr; p.norm_w_dtype = 0; p.x_out = nullptr; p.ldx = 0; p.out_sumsq = nullptr;
    p.in_sumsq = nullptr; p.in_parts = 0; p.in_inv_hidden = 0.f; p.in_eps = 0.f; p.staged_ok = 0;
    p.split_stride = 0;
    p.independent = (epilogue == TC_T_PARTIAL || epilogue == TC_T_SWIGLU) ? 0 : 1;
    p.tiles_a = (rowsA + TC_BM - 1) / TC_BM;
    p.tiles_b = (rowsB + bn - 1) / bn;
    p.splits = splits;
    const long work = (long)p.tiles_a * p.tiles_b * splits;
    if (work > 0x7fffffffL) return CML_ERR_BAD_SIZE;
    // Large tiles fill an SM: one persistent block per SM walks the items. Decode tiles are
    // small: one block per item, several per SM; but where the items are many times the SMs (the
    // output head: a thousand tiles) persistent blocks, one per SM with the deep ring, spare
    // every wave after the first its start-up (barriers, tensor memory, an empty ring).
    const int sms = cml_sm_count();
    const bool deep = bn <= 64 && p.kb_per_split >= 12;             // as launch_tc chooses
    const bool persistent = bn >= 128 || (deep && work >= 4L * sms);
    dim3 grid((unsigned)(persistent ? (work < sms ? work : sms) : work), 1, 1);
    cudaStream_t s = (cudaStream_t)stream;
#define TC_CASE(BN_, EPI_) if (bn == BN_ && epilogue == EPI_) return launch_tc<BN_, EPI_>(ma, mb, p, grid, s)
    TC_CASE(128, TC_STORE); TC_CASE(128, TC_STORE_F32); TC_CASE(128, TC_ADD_F32); TC_CASE(128, TC_SWIGLU);
    TC_CASE(256, TC_STORE); TC_CASE(256, TC_STORE_F32); TC_CASE(256, TC_ADD_F32); TC_CASE(256, TC_SWIGLU);
    TC_CASE(64, TC_STORE); TC_CASE(64, TC_STORE_F32); TC_CASE(64, TC_ADD_F32); TC_CASE(64, TC_SWIGLU);
    TC_CASE(16, TC_T_PARTIAL); TC_CASE(32, TC_T_PARTIAL); TC_CASE(64, TC_T_PARTIAL);
    TC_CASE(128, TC_T_PARTIAL);
    TC_CASE(16, TC_T_SWIGLU); TC_CASE(32, TC_T_SWIGLU); TC_CASE(64, TC_T_SWIGLU);
    TC_CASE(128, TC_T_SWIGLU);
#undef TC_CASE
    return CML_ERR_BAD_SIZE;
}

template <int EPI, int BN>
static int launch_tc_pair2(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, dim3 grid, cudaStream_t s) {
    const size_t smem = tc_pair_smem_bytes();
    cudaError_t e = cml_allow_smem<gemm_tc_pair_kernel<EPI, BN>>(smem);
    if (e != cudaSuccess) return (int)e;
    e = launch_pdl(gemm_tc_pair_kernel<EPI, BN>, grid, dim3(TC_THREADS), smem, s, ma, mb, p);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
// Tiles are 256 x 256, or 256 x 192 where that needs fewer rounds of clusters (see pair_tile_width).
// 256 x 128 was measured too: it moves as much operand data per flop as a 128 x 256 tile of one
// block and ran at little more than half the rate of 256 x 256 on every shape tried.
template <int EPI>
static int launch_tc_pair(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, int bn, dim3 grid, cudaStream_t s) {
    return bn == 192 ? launch_tc_pair2<EPI, 192>(ma, mb, p, grid, s) : launch_tc_pair2<EPI, 256>(ma, mb, p, grid, s);
}

// Columns of a tile: 192 if the rounds of `clusters` clusters it needs, times its width, are
// clearly fewer than with 256 (a narrower tile moves more operand data per flop), else 256.
static int pair_tile_width(int rowsA, int rowsB, int clusters) {
    auto cost = [&](int bn) {
        const long tiles = (long)((rowsA + 255) / 256) * ((rowsB + bn - 1) / bn);
        return ((tiles + clusters - 1) / clusters) * bn;
    };
    return cost(192) * 10 < cost(256) * 9 ? 192 : 256;
}

struct TcPairNorm {
    const void* norm_w; int norm_w_dtype; void* x_out; long ldx; float* out_sumsq;     // TC_ADD_NORM
    const float* in_sumsq; int in_parts; int in_hidden; float in_eps;                  // rows of A still lack their scale
    int splits; long split_stride;                                                     // TC_STORE_F32 split over K
};

static int gemm_tc_pair_launch(const void* A, long lda, int rowsA, const void* B, long ldb, int rowsB, int K, void* C,
                               long ldc, int epilogue, int* err, const TcPairNorm& nm, void* stream) {
    if (rowsA <= 0 || rowsB <= 0) return 0;
    if (K <= 0 || (K & 7)) return CML_ERR_BAD_SIZE;
    const int sms = cml_sm_count();
    // the norm's sums of squares are kept per 256 columns: that epilogue stays on the wide tile
    // (so does a product split over K: its splits, not a narrower tile, fill the clusters)
    const int bn = (epilogue == TC_ADD_NORM || nm.splits > 1) ? 256 : pair_tile_width(rowsA, rowsB, sms / 2);
    CUtensorMap ma, mb;
    int rc = make_map(&ma, A, rowsA, K, lda, TC_BM);
    if (rc) return rc;
    rc = make_map(&mb, B, rowsB, K, ldb, bn / 2);
    if (rc) return rc;
    TcParams p;
    p.C = C; p.ldc = ldc; p.rowsA = rowsA; p.rowsB = rowsB;
    p.num_kb = (K + TC_BK - 1) / TC_BK;
    int splits = nm.splits < 1 ? 1 : (nm.splits > p.num_kb ? p.num_kb : nm.splits);
    if (splits > 1 && epilogue != TC_STORE_F32) return CML_ERR_BAD_SIZE;
    p.kb_per_split = (p.num_kb + splits - 1) / splits;
    splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;      // no split without a k-block
    p.err = err;
    p.independent = 1;
    p.tiles_a = (rowsA + 255) / 256;
    p.tiles_b = (rowsB + bn - 1) / bn;
    p.splits = splits;
    p.split_stride = nm.split_stride;
    p.norm_w = nm.norm_w; p.norm_w_dtype = nm.norm_w_dtype; p.x_out = (bf16*)nm.x_out; p.ldx = nm.ldx;
    p.out_sumsq = nm.out_sumsq;
    p.in_sumsq = nm.in_sumsq; p.in_parts = nm.in_parts;
    p.in_inv_hidden = nm.in_hidden > 0 ? 1.0f / (float)nm.in_hidden : 0.f;
    p.in_eps = nm.in_eps;
    if (epilogue == TC_STORE) p.staged_ok = ((uintptr_t)C % 8 == 0) && (ldc % 4 == 0);
    else p.staged_ok = ((uintptr_t)C % 16 == 0) && (ldc % 4 == 0) && (nm.split_stride % 4 == 0) &&
                       (epilogue != TC_ADD_NORM || (((uintptr_t)nm.x_out % 8 == 0) && (nm.ldx % 4 == 0)));
    const long work = (long)p.tiles_a * p.tiles_b * p.splits;
    if (work > 0x7fffffffL) return CML_ERR_BAD_SIZE;
    const long clusters = work < sms / 2 ? work : sms / 2;
    dim3 grid((unsigned)(2 * clusters), 1, 1);
    cudaStream_t s = (cudaStream_t)stream;
    switch (epilogue) {
        case TC_STORE: return launch_tc_pair<TC_STORE>(ma, mb, p, bn, grid, s);
        case TC_STORE_F32: return launch_tc_pair<TC_STORE_F32>(ma, mb, p, bn, grid, s);
        case TC_ADD_F32: return launch_tc_pair<TC_ADD_F32>(ma, mb, p, bn, grid, s);
        case TC_SWIGLU: return launch_tc_pair<TC_SWIGLU>(ma, mb, p, bn, grid, s);
        case TC_ADD_NORM: return launch_tc_pair<TC_ADD_NORM>(ma, mb, p, bn, grid, s);
    }
    return CML_ERR_BAD_SIZE;
}

// The same product as cml_gemm_tc with epilogues 0..3, on tiles of 256 x 256 that two blocks
// of a cluster share (see gemm_tc_pair_kernel). For many rows of A: a tile covers 256 of them.
// in_sumsq (may be null): float [in_parts][rowsA]; the rows of A came out of a norm without
// their scale rsqrt(sum_t in_sumsq[t][row] / in_hidden + in_eps), and this product applies it
// to its output rows instead (before the SwiGLU of that epilogue).
extern "C" int cml_gemm_tc_pair(const void* A, long lda, int rowsA, const void* B, long ldb, int rowsB, int K, void* C,
                                long ldc, int epilogue, int* err, const float* in_sumsq, int in_parts, int in_hidden,
                                float in_eps, void* stream) {
    if (epilogue < TC_STORE || epilogue > TC_SWIGLU) return CML_ERR_BAD_SIZE;
    if (in_sumsq && (in_parts < 1 || in_hidden < 1)) return CML_ERR_BAD_SIZE;
    TcPairNorm nm = {nullptr, 0, nullptr, 0, nullptr, in_sumsq, in_parts, in_hidden, in_eps, 1, 0};
    return gemm_tc_pair_launch(A, lda, rowsA, B, ldb, rowsB, K, C, ldc, epilogue, err, nm, stream);
}

// The same product split over K into `splits` float partial sums: split s (k-blocks of 64 dealt
// out evenly, in order) writes C + s * split_stride; their sum over s is A B^T. For products of a
// few hundred rows, whose tiles alone would leave most of the SMs without work. `splits` must
// leave no split without a k-block: with n k-blocks, ceil(n / ceil(n / splits)) == splits.
extern "C" int cml_gemm_tc_pair_partial(const void* A, long lda, int rowsA, const void* B, long ldb, int rowsB, int K,
                                        float* C, long ldc, long split_stride, int splits, int* err,
                                        const float* in_sumsq, int in_parts, int in_hidden, float in_eps, void* stream) {
    if (splits < 1 || (in_sumsq && (in_parts < 1 || in_hidden < 1))) return CML_ERR_BAD_SIZE;
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    const int per = (num_kb + (splits > num_kb ? num_kb : splits) - 1) / (splits > num_kb ? num_kb : splits);
    if ((num_kb + per - 1) / per != splits) return CML_ERR_BAD_SIZE;
    TcPairNorm nm = {nullptr, 0, nullptr, 0, nullptr, in_sumsq, in_parts, in_hidden, in_eps, splits, split_stride};
    return gemm_tc_pair_launch(A, lda, rowsA, B, ldb, rowsB, K, C, ldc, TC_STORE_F32, err, nm, stream);
}

// C [rowsA, rowsB] float (the residual stream) += A B^T, and for the norm that reads C next:
// x_out [rowsA, rowsB] bfloat16 = C * norm_w (without the rows' scale) and out_sumsq
// [ceil(rowsB / 256)][rowsA] = the sum of squares of each row's 256 columns of a tile. The
// product that reads x_out passes out_sumsq as its in_sumsq.
extern "C" int cml_gemm_tc_pair_add_norm(const void* A, long lda, int rowsA, const void* B, long ldb, int rowsB, int K,
                                         float* C, long ldc, int* err, const void* norm_w, int norm_w_dtype,
                                         void* x_out, long ldx, float* out_sumsq, void* stream) {
    if (!norm_w || !x_out || !out_sumsq) return CML_ERR_BAD_SIZE;
    if (norm_w_dtype != CML_DTYPE_F32 && norm_w_dtype != CML_DTYPE_BF16) return CML_ERR_BAD_DTYPE;
    TcPairNorm nm = {norm_w, norm_w_dtype, x_out, ldx, out_sumsq, nullptr, 0, 0, 0.f, 1, 0};
    return gemm_tc_pair_launch(A, lda, rowsA, B, ldb, rowsB, K, C, ldc, TC_ADD_NORM, err, nm, stream);
}
