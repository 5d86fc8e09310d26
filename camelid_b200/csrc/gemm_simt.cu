// C[M, N] = A[M, K] * W[N, K]^T on the CUDA cores with float accumulation, for any M, N, K.
//
// This is the matrix product of the true 32-bit path (plain FMA, no reduced-precision
// tensor mode) and the one that takes every shape the tensor-core kernel refuses. It stands
// where the reference runs q8_gemv / q8_gemm_batched (src/cuda_resident.rs:230, :1494) with
// their fused residual add (:304-307). In the tiled forms each output element sums
// k = 0..K-1 in order wherever it lies in its tile; in the streaming form for few rows the
// order is fixed by N, K and the device's block count. Either way the value of a row does
// not depend on which other rows are in the step, only on which form the step's row count
// selects (up to 64 rows: streaming; more: tiles).
//
// Epilogues: store in the input type; store float; add into a float matrix (the residual
// stream); SwiGLU, where output column j takes weight rows gate(j) and up(j) of a packed
// [2*N, K] matrix interleaved in groups of `group` rows and stores silu(g) * u.
#include "common.cuh"
#include <cuda.h>

#define GEMM_BM 64
#define GEMM_BN 64
#define GEMM_BK 16
#define GEMM_PAD 4

enum { EPI_STORE = 0, EPI_STORE_F32 = 1, EPI_ADD_F32 = 2, EPI_SWIGLU = 3 };

template <typename T, int EPI>
__global__ void __launch_bounds__(256)
gemm_tn_simt_kernel(const T* __restrict__ A, int lda, const T* __restrict__ W, int ldw, void* __restrict__ Cv,
                    int ldc, int M, int N, int K, int group) {
    __shared__ __align__(16) float As[GEMM_BK][GEMM_BM + GEMM_PAD];
    __shared__ __align__(16) float Ws[GEMM_BK][GEMM_BN + GEMM_PAD];
    __shared__ __align__(16) float Us[EPI == EPI_SWIGLU ? GEMM_BK : 1][GEMM_BN + GEMM_PAD];
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * GEMM_BM, n0 = blockIdx.x * GEMM_BN;
    const int lr = tid >> 2;            // 0..63: tile row loaded by this thread
    const int lk = (tid & 3) * 4;       // first of its 4 consecutive k

    float acc[4][4], acc2[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f, acc2[i][j] = 0.f;

    const int arow = m0 + lr;
    const int wcol = n0 + lr;
    long wrow = wcol, urow = 0;
    if (EPI == EPI_SWIGLU) {
        wrow = (long)(wcol / group) * 2 * group + wcol % group;
        urow = wrow + group;
    }
    for (int k0 = 0; k0 < K; k0 += GEMM_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            const bool kin = k < K;
            As[lk + i][lr] = (kin && arow < M) ? to_f32(A[(size_t)arow * lda + k]) : 0.f;
            Ws[lk + i][lr] = (kin && wcol < N) ? to_f32(W[(size_t)wrow * ldw + k]) : 0.f;
            if (EPI == EPI_SWIGLU) Us[lk + i][lr] = (kin && wcol < N) ? to_f32(W[(size_t)urow * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GEMM_BK; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w};
            const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
            if (EPI == EPI_SWIGLU) {
                const float4 u = *reinterpret_cast<const float4*>(&Us[k][tx * 4]);
                const float uv[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc2[i][j] = fmaf(av[i], uv[j], acc2[i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = m0 + ty * 4 + i;
        if (r >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = n0 + tx * 4 + j;
            if (c >= N) continue;
            const size_t o = (size_t)r * ldc + c;
            if (EPI == EPI_STORE) ((T*)Cv)[o] = from_f32<T>(acc[i][j]);
            else if (EPI == EPI_STORE_F32) ((float*)Cv)[o] = acc[i][j];
            else if (EPI == EPI_ADD_F32) ((float*)Cv)[o] += acc[i][j];
            else {
                const float g = acc[i][j];
                ((T*)Cv)[o] = from_f32<T>((g / (1.0f + expf(-g))) * acc2[i][j]);
            }
        }
    }
}

// Many rows in float: tiles of 128 x 128 outputs, 256 threads with 8 x 8 outputs each, K in steps of 16
// through two shared-memory buffers (the next step's operands are fetched into registers, 16 bytes at a
// time, while this step is multiplied). Both operands are kept transposed in shared memory, so a thread
// reads its 8 rows and 8 columns as two 16-byte pieces each. A thread's columns are two groups of four, 16
// apart: on a packed gate/up matrix interleaved in groups of 16 those are four gate rows and the up rows
// of the same outputs, so SwiGLU needs no second accumulator. Every output still sums k = 0..K-1 in order.
// Needs K and the row strides in multiples of 4 floats and 16-byte aligned operands; other sizes and types
// take the 64 x 64 kernel above.
#define GB_M 128
#define GB_N 128
#define GB_K 16
#define GB_LD (GB_M + 4)
// Columns of the weight tile are kept with their 16-byte pieces permuted (piece p of the second half of every
// 32 columns at p ^ 4), so that the eight lanes of a quarter warp, which read pieces {0..3, 8..11} (+4 for the
// second group), touch eight different sets of four banks.
__device__ __forceinline__ int gb_wcol(int c) { return c ^ (((c >> 5) & 1) << 4); }
template <int EPI>
__global__ void __launch_bounds__(256, 2)
gemm_tn_f32_big_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw, float* __restrict__ C,
                       int ldc, int M, int n_wrows, int K) {
    __shared__ __align__(16) float As[2][GB_K][GB_LD];
    __shared__ __align__(16) float Ws[2][GB_K][GB_LD];
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * GB_M, n0 = blockIdx.x * GB_N;
    // this thread's output columns within the tile: two groups of four, 16 apart
    const int cg = (tx >> 2) * 32 + (tx & 3) * 4;
    // the two 16-byte pieces of each operand tile this thread fetches per step
    const int lrow0 = tid >> 2, lrow1 = lrow0 + 64, lkq = (tid & 3) * 4;
    const int wcol0 = gb_wcol(lrow0), wcol1 = gb_wcol(lrow1);
    const int cg0 = gb_wcol(cg), cg1 = gb_wcol(cg + 16);
    const float* a0p = A + (size_t)min(m0 + lrow0, M - 1) * lda + lkq;
    const float* a1p = A + (size_t)min(m0 + lrow1, M - 1) * lda + lkq;
    const float* w0p = W + (size_t)min(n0 + lrow0, n_wrows - 1) * ldw + lkq;
    const float* w1p = W + (size_t)min(n0 + lrow1, n_wrows - 1) * ldw + lkq;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    // a thread's 8 x 8 sums as pairs of neighbouring columns: one packed FMA (two IEEE float FMAs in one
    // instruction, sm_100) per pair and k, half the instructions and register reads of single FMAs
    float2 acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = make_float2(0.f, 0.f);

    auto fetch = [&](int k0, float4& ra0, float4& ra1, float4& rw0, float4& rw1) {
        const bool in = k0 + lkq < K;
        ra0 = in ? *reinterpret_cast<const float4*>(a0p + k0) : zero;
        ra1 = in ? *reinterpret_cast<const float4*>(a1p + k0) : zero;
        rw0 = in ? *reinterpret_cast<const float4*>(w0p + k0) : zero;
        rw1 = in ? *reinterpret_cast<const float4*>(w1p + k0) : zero;
    };
    auto stash = [&](int buf, const float4& ra0, const float4& ra1, const float4& rw0, const float4& rw1) {
        As[buf][lkq + 0][lrow0] = ra0.x; As[buf][lkq + 1][lrow0] = ra0.y; As[buf][lkq + 2][lrow0] = ra0.z; As[buf][lkq + 3][lrow0] = ra0.w;
        As[buf][lkq + 0][lrow1] = ra1.x; As[buf][lkq + 1][lrow1] = ra1.y; As[buf][lkq + 2][lrow1] = ra1.z; As[buf][lkq + 3][lrow1] = ra1.w;
        Ws[buf][lkq + 0][wcol0] = rw0.x; Ws[buf][lkq + 1][wcol0] = rw0.y; Ws[buf][lkq + 2][wcol0] = rw0.z; Ws[buf][lkq + 3][wcol0] = rw0.w;
        Ws[buf][lkq + 0][wcol1] = rw1.x; Ws[buf][lkq + 1][wcol1] = rw1.y; Ws[buf][lkq + 2][wcol1] = rw1.z; Ws[buf][lkq + 3][wcol1] = rw1.w;
    };
    float4 ra0, ra1, rw0, rw1;
    fetch(0, ra0, ra1, rw0, rw1);
    stash(0, ra0, ra1, rw0, rw1);
    __syncthreads();
    const int steps = (K + GB_K - 1) / GB_K;
    for (int st = 0; st < steps; ++st) {
        const int buf = st & 1;
        if (st + 1 < steps) fetch((st + 1) * GB_K, ra0, ra1, rw0, rw1);
#pragma unroll
        for (int k = 0; k < GB_K; ++k) {
            const float4 av0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 8]);
            const float4 av1 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 8 + 4]);
            const float4 bv0 = *reinterpret_cast<const float4*>(&Ws[buf][k][cg0]);
            const float4 bv1 = *reinterpret_cast<const float4*>(&Ws[buf][k][cg1]);
            const float av[8] = {av0.x, av0.y, av0.z, av0.w, av1.x, av1.y, av1.z, av1.w};
            const float2 bv[4] = {make_float2(bv0.x, bv0.y), make_float2(bv0.z, bv0.w), make_float2(bv1.x, bv1.y),
                                  make_float2(bv1.z, bv1.w)};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 a2 = make_float2(av[i], av[i]);
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = __ffma2_rn(a2, bv[j], acc[i][j]);
            }
        }
        if (st + 1 < steps) {
            stash(buf ^ 1, ra0, ra1, rw0, rw1);      // the other buffer was last read a step ago, before the barrier below
            __syncthreads();
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = m0 + ty * 8 + i;
        if (r >= M) continue;
        if (EPI == EPI_SWIGLU) {
            // columns cg..cg+3 are gate rows, cg+16.. the up rows of the same outputs (interleave groups of 16)
            const int out0 = (n0 + cg - (tx & 3) * 4) / 2 + (tx & 3) * 4;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = out0 + j;
                if (2 * c < n_wrows) {
                    const float g = (j & 1) ? acc[i][j >> 1].y : acc[i][j >> 1].x;
                    const float u = (j & 1) ? acc[i][2 + (j >> 1)].y : acc[i][2 + (j >> 1)].x;
                    C[(size_t)r * ldc + c] = (g / (1.0f + expf(-g))) * u;
                }
            }
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int c = n0 + cg + 16 * h + j;
                    if (c >= n_wrows) continue;
                    float* o = C + (size_t)r * ldc + c;
                    const float v = (j & 1) ? acc[i][2 * h + (j >> 1)].y : acc[i][2 * h + (j >> 1)].x;
                    if (EPI == EPI_ADD_F32) *o += v;
                    else *o = v;
                }
        }
    }
}

static int launch_gemm_f32_big(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
                               int epilogue, cudaStream_t s) {
    const int n_wrows = epilogue == EPI_SWIGLU ? 2 * N : N;
    dim3 grid((n_wrows + GB_N - 1) / GB_N, (M + GB_M - 1) / GB_M);
    if (grid.y > 65535) return CML_ERR_BAD_SIZE;
#define CML_GEMMB(E) launch_pdl(gemm_tn_f32_big_kernel<E>, grid, dim3(256), 0, s, (const float*)A, lda, (const float*)W, ldw, (float*)C, ldc, M, n_wrows, K)
    switch (epilogue) {
        case EPI_STORE:
        case EPI_STORE_F32: CML_GEMMB(EPI_STORE_F32); break;
        case EPI_ADD_F32: CML_GEMMB(EPI_ADD_F32); break;
        case EPI_SWIGLU: CML_GEMMB(EPI_SWIGLU); break;
        default: return CML_ERR_BAD_SIZE;
    }
#undef CML_GEMMB
    return cml_launch_status();
}

// Few rows in float, the plain form (any K, any alignment, any interleave group): every output column is one warp's dot products, the weight row
// read once with 16-byte loads and used for all MB activation rows, which stay in cache.
// Each lane sums its k's in ascending order, then the lanes are summed in a fixed tree: the
// value of a row does not depend on the other rows of the step.
template <int MB, int EPI>
__global__ void __launch_bounds__(256)
gemv_f32_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw, float* __restrict__ C,
                int ldc, int M, int N, int K, int group) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int m0 = blockIdx.y * MB;
    if (n >= N) return;
    long wrow = n, urow = 0;
    if (EPI == EPI_SWIGLU) {
        wrow = (long)(n / group) * 2 * group + n % group;
        urow = wrow + group;
    }
    const float* wr = W + (size_t)wrow * ldw;
    const float* ur = W + (size_t)urow * ldw;
    float acc[MB], acc2[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) acc[m] = 0.f, acc2[m] = 0.f;
    const bool vec = ((K & 3) == 0) && ((lda & 3) == 0) && ((ldw & 3) == 0) && (((uintptr_t)A & 15) == 0) &&
                     (((uintptr_t)W & 15) == 0);
    if (vec) {
        // Four steps of 128 columns at a time: the weight loads of all four are issued before the
        // first use (they come from HBM; the activations come from cache), and no row is skipped
        // by a branch (rows beyond M repeat the last row and are not stored), so nothing keeps
        // the compiler from having them in flight together.
        for (int k0 = lane * 4; k0 < K; k0 += 512) {
            float4 w4[4], u4[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int k = min(k0 + j * 128, K - 4);
                w4[j] = *reinterpret_cast<const float4*>(wr + k);
                u4[j] = EPI == EPI_SWIGLU ? *reinterpret_cast<const float4*>(ur + k) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int k = k0 + j * 128;
                if (k >= K) {                      // past the end: the clamped load above does not count
                    w4[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                    u4[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
                const int kc = min(k, K - 4);
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    const float4 a4 = *reinterpret_cast<const float4*>(A + (size_t)min(m0 + m, M - 1) * lda + kc);
                    acc[m] = fmaf(a4.x, w4[j].x, acc[m]); acc[m] = fmaf(a4.y, w4[j].y, acc[m]);
                    acc[m] = fmaf(a4.z, w4[j].z, acc[m]); acc[m] = fmaf(a4.w, w4[j].w, acc[m]);
                    if (EPI == EPI_SWIGLU) {
                        acc2[m] = fmaf(a4.x, u4[j].x, acc2[m]); acc2[m] = fmaf(a4.y, u4[j].y, acc2[m]);
                        acc2[m] = fmaf(a4.z, u4[j].z, acc2[m]); acc2[m] = fmaf(a4.w, u4[j].w, acc2[m]);
                    }
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            const float wv = wr[k];
            const float uv = EPI == EPI_SWIGLU ? ur[k] : 0.f;
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                if (m0 + m >= M) break;
                const float av = A[(size_t)(m0 + m) * lda + k];
                acc[m] = fmaf(av, wv, acc[m]);
                if (EPI == EPI_SWIGLU) acc2[m] = fmaf(av, uv, acc2[m]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MB; ++m) {
        const float v = warp_sum(acc[m]);
        const float v2 = EPI == EPI_SWIGLU ? warp_sum(acc2[m]) : 0.f;
        if (lane == 0 && m0 + m < M) {
            float* o = C + (size_t)(m0 + m) * ldc + n;
            if (EPI == EPI_ADD_F32) *o += v;
            else if (EPI == EPI_SWIGLU) *o = (v / (1.0f + expf(-v))) * v2;
            else *o = v;
        }
    }
}

// Few rows in float, the form that streams weights: a block owns tiles of 32 consecutive weight rows; every
// warp walks COLS weight rows at a time against the MB rows of the step, so an activation read from shared
// memory serves COLS dot products. Lanes take their k's in ascending order and are summed in a fixed tree
// (a butterfly that leaves sum i in lane i).
// SwiGLU needs interleave groups of 16, so that a tile of 32 packed rows is 16 gate rows and the 16 up rows
// of the same outputs.
#define GV_WARPS 8
#define GV_ROWS 32          // weight rows per tile
#define GV_MAX_ROWS 64      // steps of up to this many rows take this form, 8 rows a block: beyond it the weights' way
                            // into the SMs, once per group of 8 rows, costs more than the tiles of the many-row form
// The weights come by TMA (cp.async.bulk.tensor into a ring of shared-memory stages, completion on
// mbarriers), not by loads into registers: what a block
// has on its way from HBM is the ring (RG_STAGES stages of 32 weight rows x 128 columns, 16 KB each, two
// blocks per SM), not what its lanes can hold. A stage also carries the MB activation rows of its 128
// columns, so a block can work on any range of K. The work of a product, tiles x steps of 128
// columns, is dealt out evenly: block b takes the steps [b T / G, (b + 1) T / G) of the T steps
// in tile order, so a tile's K may be shared by two or more blocks, which leave their sums in
// `scratch` (slot tile + block) and count themselves at the tile's ticket; the block that arrives
// last adds the slots in block order (ascending k) and runs the epilogue. The order of summation
// is fixed by N, K and the number of blocks (twice the SMs of the device, or T if that is less),
// not by the number of rows: every group of 8 rows is dealt out the same way.
// Warps 0-7 compute (4 weight rows each), warp 8 issues the copies: the weights of the first
// stages before the wait on the previous kernel, their activations after it. Every wait on a
// barrier is bounded: a wait that runs out sets *err, the blocks's warps see the flag, let the
// copies in flight land and leave.
#define RG_STAGES 5
#define RG_KS 128
#define RG_WAIT_CYCLES 2000000000ll
__device__ __forceinline__ uint32_t rg_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool rg_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool rg_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (rg_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (rg_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > RG_WAIT_CYCLES) {
            *abort_flag = 1;
            return false;
        }
    }
}
__device__ __forceinline__ void rg_tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y) : "memory");
}

struct RgShape {
    int M, n_wrows, K;
    int tiles, steps;            // 32-row tiles of the weights; steps of 128 columns in K
    int blocks;                  // blocks per group of MB rows
    int splits;                  // 0: the steps dealt out evenly. Else block b owns range b % splits of the K of
    int per;                     //    tile b / splits (`per` steps a range) and stores its sums as partial sums
    long split_stride;           //    at C + range * split_stride: no tickets, the reader adds the ranges.
};
// first step of block b of the group: floor(b * T / G)
__device__ __forceinline__ int rg_first_step(const RgShape& sh, int b) {
    if (sh.splits > 0) {
        const int tile = b / sh.splits, range = b - tile * sh.splits;
        return tile * sh.steps + min(sh.steps, range * sh.per);
    }
    return (int)(((long)b * ((long)sh.tiles * sh.steps)) / sh.blocks);
}
// the block whose range holds step q: the largest b with first_step(b) <= q
__device__ __forceinline__ int rg_block_of(const RgShape& sh, int q) {
    const long T = (long)sh.tiles * sh.steps;
    int b = (int)min((long)sh.blocks - 1, (((long)q + 1) * sh.blocks - 1) / T);
    while (b > 0 && rg_first_step(sh, b) > q) --b;
    while (b + 1 < sh.blocks && rg_first_step(sh, b + 1) <= q) ++b;
    return b;
}

template <int MB, int EPI>
__global__ void __launch_bounds__((GV_WARPS + 1) * 32, 2)
gemv_f32_ring_kernel(const __grid_constant__ CUtensorMap mapW, const __grid_constant__ CUtensorMap mapA, float* __restrict__ C,
                     int ldc, RgShape sh, float* __restrict__ scratch, int* __restrict__ tickets, int* err) {
    constexpr int COLS = GV_ROWS / GV_WARPS;
    constexpr int STAGE_FLOATS = (GV_ROWS + MB) * RG_KS;
    extern __shared__ __align__(128) float ring[];               // [RG_STAGES][GV_ROWS + MB][RG_KS]
    __shared__ float sums[MB * GV_ROWS];
    __shared__ __align__(8) uint64_t bars[2 * RG_STAGES];
    __shared__ int s_last;
    __shared__ int s_abort;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int b = blockIdx.x, group = blockIdx.y;
    const int m0 = group * MB;
    const int q_lo = rg_first_step(sh, b), q_hi = rg_first_step(sh, b + 1);
    const uint32_t full0 = rg_smem_u32(bars), empty0 = full0 + 8u * RG_STAGES;
    volatile int* abort_flag = &s_abort;
    if (threadIdx.x == 0) {
        for (int s = 0; s < RG_STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full0 + 8u * s), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty0 + 8u * s), "r"(GV_WARPS));
        }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == GV_WARPS) {
        // producer: stage (q - q_lo) % RG_STAGES holds step q
        const uint32_t ring_u32 = rg_smem_u32(ring);
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&mapW) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&mapA) : "memory");
        }
        auto issue = [&](int q, bool weights, bool acts) {
            if (lane != 0) return;
            const int tile = q / sh.steps, ks = q - tile * sh.steps;
            const int s = (q - q_lo) % RG_STAGES;
            const uint32_t dst = ring_u32 + (uint32_t)s * STAGE_FLOATS * 4u, bar = full0 + 8u * s;
            if (weights) {
                // parts of a box beyond the matrix arrive as zeros and count as bytes all the same
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)STAGE_FLOATS * 4u) : "memory");
                rg_tma_load_2d(dst, &mapW, bar, ks * RG_KS, tile * GV_ROWS);
            }
            if (acts) rg_tma_load_2d(dst + (uint32_t)GV_ROWS * RG_KS * 4u, &mapA, bar, ks * RG_KS, m0);
        };
        const int q_pre = min(q_hi, q_lo + RG_STAGES);
        for (int q = q_lo; q < q_pre; ++q) issue(q, true, false);
        pdl_wait();
        for (int q = q_lo; q < q_pre; ++q) issue(q, false, true);
        bool ok = true;
        int q = q_pre;
        for (; q < q_hi; ++q) {
            const int i = q - q_lo;
            ok = rg_wait(empty0 + 8u * (uint32_t)(i % RG_STAGES), (uint32_t)((i / RG_STAGES) - 1) & 1u, abort_flag);
            if (!ok) break;
            issue(q, true, true);
        }
        // The warp stays until what it issued has landed (the block's shared memory must outlive its copies).
        for (int j = max(q_lo, q - RG_STAGES); j < q; ++j) {
            const int i = j - q_lo;
            const long long t0 = clock64();
            while (!rg_try_wait(full0 + 8u * (uint32_t)(i % RG_STAGES), (uint32_t)(i / RG_STAGES) & 1u) &&
                   clock64() - t0 < (*abort_flag ? 20000000ll : RG_WAIT_CYCLES)) {}
        }
        if (*abort_flag && lane == 0) atomicExch(err, 8);
        return;
    }

    // consumers
    pdl_wait();
    const int tid = threadIdx.x;                                   // 0 .. 255
    int q = q_lo;
    while (q < q_hi) {
        const int tile = q / sh.steps;
        const int tile_q0 = tile * sh.steps;
        const int q_end = min(q_hi, tile_q0 + sh.steps);
        float acc[MB][COLS];
#pragma unroll
        for (int m = 0; m < MB; ++m)
#pragma unroll
            for (int c = 0; c < COLS; ++c) acc[m][c] = 0.f;
        bool ok = true;
        for (; q < q_end; ++q) {
            const int i = q - q_lo;
            const int s = i % RG_STAGES;
            ok = rg_wait(full0 + 8u * (uint32_t)s, (uint32_t)(i / RG_STAGES) & 1u, abort_flag);
            if (!ok) break;
            const float* st = ring + (size_t)s * STAGE_FLOATS;
            {
                float4 w4[COLS];
#pragma unroll
                for (int c = 0; c < COLS; ++c) w4[c] = *reinterpret_cast<const float4*>(st + (warp * COLS + c) * RG_KS + lane * 4);
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    const float4 a4 = *reinterpret_cast<const float4*>(st + (GV_ROWS + m) * RG_KS + lane * 4);
#pragma unroll
                    for (int c = 0; c < COLS; ++c) {
                        acc[m][c] = fmaf(a4.x, w4[c].x, acc[m][c]); acc[m][c] = fmaf(a4.y, w4[c].y, acc[m][c]);
                        acc[m][c] = fmaf(a4.z, w4[c].z, acc[m][c]); acc[m][c] = fmaf(a4.w, w4[c].w, acc[m][c]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty0 + 8u * (uint32_t)s) : "memory");
        }
        if (!ok) q = q_hi;                                         // no more steps; the barriers below are still kept
        {   // the warp's 32 sums over its lanes, 31 shuffles in all: lane i ends up with sum i = acc[i / 4][i % 4]
            float v[MB * COLS];
#pragma unroll
            for (int m = 0; m < MB; ++m)
#pragma unroll
                for (int c = 0; c < COLS; ++c) v[m * COLS + c] = acc[m][c];
            static_assert(MB * COLS == 32, "one sum per lane");
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) {
                const bool upper = (lane & off) != 0;          // keeps the upper half of what is left, sends the lower
#pragma unroll
                for (int i = 0; i < off; ++i) {
                    const float send = upper ? v[i] : v[i + off];
                    const float keep = upper ? v[i + off] : v[i];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
            sums[(lane / COLS) * GV_ROWS + warp * COLS + (lane % COLS)] = v[0];
        }
        {   // one answer for all eight warps: has any of them, or the producer, given up?
            uint32_t stop;
            asm volatile(
                "{\n\t.reg .pred p, q;\n\t"
                "setp.ne.u32 q, %1, 0;\n\t"
                "bar.red.or.pred p, 1, 256, q;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(stop) : "r"((uint32_t)(!ok || *abort_flag)) : "memory");
            if (stop) {
                if (tid == 0) atomicExch(err, 8);
                break;
            }
        }
        const int t_in = tile % sh.tiles;                          // tile within the group
        if (sh.splits > 0) {                                       // this range's sums, as they are
            float* part = C + (size_t)(b - tile * sh.splits) * sh.split_stride;
            for (int i = tid; i < MB * GV_ROWS; i += 256) {
                const int m = i / GV_ROWS, j = i - m * GV_ROWS;
                const int n = t_in * GV_ROWS + j;
                if (m0 + m < sh.M && n < sh.n_wrows) part[(size_t)(m0 + m) * ldc + n] = sums[i];
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            continue;
        }
        const int b_first = rg_block_of(sh, tile_q0), b_last = rg_block_of(sh, tile_q0 + sh.steps - 1);
        bool mine = true;                                          // does this block run the tile's epilogue?
        if (b_last > b_first) {
            const size_t slots = (size_t)sh.tiles + sh.blocks;
            float* slot = scratch + ((size_t)group * slots + t_in + b) * (MB * GV_ROWS);
            for (int i = tid; i < MB * GV_ROWS; i += 256) slot[i] = sums[i];
            __threadfence();
            asm volatile("bar.sync 1, 256;" ::: "memory");
            int* ticket = tickets + (size_t)group * sh.tiles + t_in;
            if (tid == 0) {
                const int t = atomicAdd(ticket, 1);
                s_last = (t == b_last - b_first);
                if (s_last) *ticket = 0;                           // left zero for the next launch
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            mine = s_last != 0;
            if (mine) {
                __threadfence();
                const float* all = scratch + ((size_t)group * slots + t_in) * (MB * GV_ROWS);
                for (int i = tid; i < MB * GV_ROWS; i += 256) {
                    float v = 0.f;
                    for (int bb = b_first; bb <= b_last; ++bb) v += __ldcg(all + (size_t)bb * (MB * GV_ROWS) + i);
                    sums[i] = v;
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");
            }
        }
        if (mine) {
            if (EPI == EPI_SWIGLU) {
                for (int i = tid; i < MB * (GV_ROWS / 2); i += 256) {
                    const int m = i / (GV_ROWS / 2), j = i - m * (GV_ROWS / 2);
                    const int n = t_in * (GV_ROWS / 2) + j;
                    if (m0 + m < sh.M && 2 * n < sh.n_wrows) {
                        const float g = sums[m * GV_ROWS + j], u = sums[m * GV_ROWS + GV_ROWS / 2 + j];
                        C[(size_t)(m0 + m) * ldc + n] = (g / (1.0f + expf(-g))) * u;
                    }
                }
            } else {
                for (int i = tid; i < MB * GV_ROWS; i += 256) {
                    const int m = i / GV_ROWS, j = i - m * GV_ROWS;
                    const int n = t_in * GV_ROWS + j;
                    if (m0 + m < sh.M && n < sh.n_wrows) {
                        float* o = C + (size_t)(m0 + m) * ldc + n;
                        if (EPI == EPI_ADD_F32) *o += sums[i];
                        else *o = sums[i];
                    }
                }
            }
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");             // sums is free for the next tile
    }
}

// Scratch the streaming form needs: tickets (ints, kept zero) in a first part of fixed size, which products of
// every shape share, then one slot of MB x 32 sums per (tile + block) of each group of 8 rows. A step has at
// most 8 groups; GV_TICKETS tickets cover a quarter of a million weight rows at eight groups; more are refused.
#define GV_TICKETS 65536
static RgShape rg_shape(int M, int n_wrows, int K) {
    RgShape sh;
    sh.M = M; sh.n_wrows = n_wrows; sh.K = K;
    sh.tiles = (n_wrows + GV_ROWS - 1) / GV_ROWS;
    sh.steps = (K + RG_KS - 1) / RG_KS;
    const long T = (long)sh.tiles * sh.steps;
    sh.blocks = (int)min((long)2 * cml_sm_count(), T);       // two blocks per SM: all of its shared memory as rings
    sh.splits = 0; sh.per = 0; sh.split_stride = 0;
    return sh;
}

extern "C" long cml_gemv_f32_scratch_bytes(int M, int N, int K, int epilogue) {
    const int n_wrows = epilogue == EPI_SWIGLU ? 2 * N : N;
    const int groups = (M + 7) / 8;
    const RgShape sh = rg_shape(M, n_wrows, K);
    return (long)GV_TICKETS * sizeof(int) + (long)groups * ((long)sh.tiles + sh.blocks) * 8 * GV_ROWS * (long)sizeof(float);
}

typedef CUresult (*RgEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static RgEncodeFn rg_encode_fn() {
    static RgEncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (RgEncodeFn)p;
    }
    return fn;
}
// A map over a row-major float matrix [rows, K] (row stride ld elements): boxes of 128 columns by box_rows
// rows, rows as they lie (no swizzle); what a box holds beyond the matrix reads as zero.
static int rg_make_map(CUtensorMap* map, const void* base, long rows, long K, long ld, int box_rows) {
    RgEncodeFn fn = rg_encode_fn();
    if (!fn) return CML_ERR_BAD_SIZE;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
    cuuint32_t box[2] = {RG_KS, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : CML_ERR_BAD_SIZE;
}

static int launch_gemv_f32_ring(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
                                int epilogue, void* scratch, int* err, cudaStream_t s) {
    constexpr int MB = 8;
    const int n_wrows = epilogue == EPI_SWIGLU ? 2 * N : N;
    const int groups = (M + MB - 1) / MB;
    const RgShape sh = rg_shape(M, n_wrows, K);
    if ((long)sh.tiles * groups > GV_TICKETS || (long)sh.tiles * sh.steps > 0x7fffffffL) return CML_ERR_BAD_SIZE;
    CUtensorMap mw, ma;
    int rc = rg_make_map(&mw, W, n_wrows, K, ldw, GV_ROWS);
    if (rc) return rc;
    rc = rg_make_map(&ma, A, M, K, lda, MB);
    if (rc) return rc;
    const size_t smem = (size_t)RG_STAGES * (GV_ROWS + MB) * RG_KS * sizeof(float);
    int* tickets = (int*)scratch;
    float* sums = (float*)((char*)scratch + (size_t)GV_TICKETS * sizeof(int));
    dim3 grid(sh.blocks, groups);
    cudaError_t e;
#define CML_GEMVR(E)                                                                                                    \
    e = cml_allow_smem<gemv_f32_ring_kernel<MB, E>>(smem);                                                              \
    if (e != cudaSuccess) return (int)e;                                                                                \
    launch_pdl(gemv_f32_ring_kernel<MB, E>, grid, dim3((GV_WARPS + 1) * 32), smem, s, mw, ma, (float*)C, ldc, sh, sums, \
               tickets, err)
    switch (epilogue) {
        case EPI_STORE:
        case EPI_STORE_F32: CML_GEMVR(EPI_STORE_F32); break;
        case EPI_ADD_F32: CML_GEMVR(EPI_ADD_F32); break;
        case EPI_SWIGLU: CML_GEMVR(EPI_SWIGLU); break;
        default: return CML_ERR_BAD_SIZE;
    }
#undef CML_GEMVR
    return cml_launch_status();
}

// Ranges of K a product of at most 64 float rows is cut into when its sums are left as partial sums: about as
// many blocks as the device holds at a time (two per SM), ranges of at least two steps of 128 columns; 0 where
// the sizes do not suit the streaming form.
extern "C" int cml_gemv_f32_partial_splits(int M, int N, int K, int lda, int ldw) {
    if (M < 1 || M > GV_MAX_ROWS || N < 1 || K < 256 || (K & 3) || (lda & 3) || (ldw & 3)) return 0;
    const int tiles = (N + GV_ROWS - 1) / GV_ROWS, steps = (K + RG_KS - 1) / RG_KS;
    int splits = max(1, min(2 * cml_sm_count() / tiles, steps / 2));
    const int per = (steps + splits - 1) / splits;
    return (steps + per - 1) / per;                                    // no empty range
}

// part[r][m][n] (float, row stride ldc, ranges split_stride apart) = the sum of A[m][k] * W[n][k] over range r of K,
// for r < splits = cml_gemv_f32_partial_splits(...). At most 64 rows (groups of 8 on blocks of their own).
extern "C" int cml_gemv_f32_partial(const void* A, int lda, const void* W, int ldw, void* part, int ldc, long split_stride,
                                    int splits, int M, int N, int K, int* err, void* stream) {
    constexpr int MB = 8;
    if (splits < 1 || splits != cml_gemv_f32_partial_splits(M, N, K, lda, ldw) || err == nullptr) return CML_ERR_BAD_SIZE;
    if ((((uintptr_t)A | (uintptr_t)W) & 15) != 0) return CML_ERR_BAD_ALIGN;
    RgShape sh = rg_shape(M, N, K);
    sh.splits = splits;
    sh.per = (sh.steps + splits - 1) / splits;
    sh.split_stride = split_stride;
    sh.blocks = sh.tiles * splits;
    CUtensorMap mw, ma;
    int rc = rg_make_map(&mw, W, N, K, ldw, GV_ROWS);
    if (rc) return rc;
    rc = rg_make_map(&ma, A, M, K, lda, MB);
    if (rc) return rc;
    const size_t smem = (size_t)RG_STAGES * (GV_ROWS + MB) * RG_KS * sizeof(float);
    cudaError_t e = cml_allow_smem<gemv_f32_ring_kernel<MB, EPI_STORE_F32>>(smem);
    if (e != cudaSuccess) return (int)e;
    launch_pdl(gemv_f32_ring_kernel<MB, EPI_STORE_F32>, dim3(sh.blocks, (M + MB - 1) / MB), dim3((GV_WARPS + 1) * 32), smem,
               (cudaStream_t)stream, mw, ma, (float*)part, ldc, sh, (float*)nullptr, (int*)nullptr, err);
    return cml_launch_status();
}

static int launch_gemv_f32(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
                           int epilogue, int group, cudaStream_t s) {
    constexpr int MB = 8;
    dim3 grid((N + 7) / 8, (M + MB - 1) / MB);
#define CML_GEMV(E) launch_pdl(gemv_f32_kernel<MB, E>, grid, dim3(256), 0, s, (const float*)A, lda, (const float*)W, ldw, (float*)C, ldc, M, N, K, group)
    switch (epilogue) {
        case EPI_STORE:
        case EPI_STORE_F32: CML_GEMV(EPI_STORE_F32); break;
        case EPI_ADD_F32: CML_GEMV(EPI_ADD_F32); break;
        case EPI_SWIGLU:
            if (group <= 0 || N % group != 0) return CML_ERR_BAD_SIZE;
            CML_GEMV(EPI_SWIGLU);
            break;
        default: return CML_ERR_BAD_SIZE;
    }
#undef CML_GEMV
    return cml_launch_status();
}

template <typename T>
static int launch_gemm(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
                       int epilogue, int group, cudaStream_t s) {
    dim3 grid((N + GEMM_BN - 1) / GEMM_BN, (M + GEMM_BM - 1) / GEMM_BM);
    if (grid.y > 65535) return CML_ERR_BAD_SIZE;
#define CML_GEMM(E) launch_pdl(gemm_tn_simt_kernel<T, E>, grid, dim3(256), 0, s, (const T*)A, lda, (const T*)W, ldw, C, ldc, M, N, K, group)
    switch (epilogue) {
        case EPI_STORE: CML_GEMM(EPI_STORE); break;
        case EPI_STORE_F32: CML_GEMM(EPI_STORE_F32); break;
        case EPI_ADD_F32: CML_GEMM(EPI_ADD_F32); break;
        case EPI_SWIGLU:
            if (group <= 0 || N % group != 0) return CML_ERR_BAD_SIZE;
            CML_GEMM(EPI_SWIGLU);
            break;
        default: return CML_ERR_BAD_SIZE;
    }
#undef CML_GEMM
    return cml_launch_status();
}

// A: [M, K] (row stride lda), W: [N, K] (or [2N, K] for SwiGLU; row stride ldw), C: [M, N] (ldc).
// `scratch` (may be null): device memory of at least cml_gemv_f32_scratch_bytes(M, N, K, epilogue) bytes whose
// first part (the tickets) is zero before the first call and left zero; with it and `err` (set to 8 if a bounded
// wait of that form runs out), float products of at most 64 rows whose sizes allow 16-byte loads take the
// streaming form.
extern "C" int cml_gemm_tn_simt(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
                                int dtype, int epilogue, int group, void* scratch, int* err, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CML_DTYPE_F32 && M <= GV_MAX_ROWS && scratch != nullptr && err != nullptr && K >= 128 && (K & 3) == 0 && (lda & 3) == 0 &&
        (ldw & 3) == 0 && (((uintptr_t)A | (uintptr_t)W) & 15) == 0 &&
        (epilogue != EPI_SWIGLU || (group == GV_ROWS / 2 && N % (GV_ROWS / 2) == 0)))
        return launch_gemv_f32_ring(A, lda, W, ldw, C, ldc, M, N, K, epilogue, scratch, err, s);
    if (dtype == CML_DTYPE_F32 && M <= 32) return launch_gemv_f32(A, lda, W, ldw, C, ldc, M, N, K, epilogue, group, s);
    if (dtype == CML_DTYPE_F32 && M > GV_MAX_ROWS && (K & 3) == 0 && (lda & 3) == 0 && (ldw & 3) == 0 &&
        (((uintptr_t)A | (uintptr_t)W) & 15) == 0 && (epilogue != EPI_SWIGLU || (group == 16 && N % 16 == 0)))
        return launch_gemm_f32_big(A, lda, W, ldw, C, ldc, M, N, K, epilogue, s);
    if (dtype == CML_DTYPE_F32) return launch_gemm<float>(A, lda, W, ldw, C, ldc, M, N, K, epilogue, group, s);
    if (dtype == CML_DTYPE_BF16) return launch_gemm<bf16>(A, lda, W, ldw, C, ldc, M, N, K, epilogue, group, s);
    return CML_ERR_BAD_DTYPE;
}
