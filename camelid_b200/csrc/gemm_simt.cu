// C[M, N] = A[M, K] * W[N, K]^T on the CUDA cores with float accumulation, for any M, N, K.
//
// This is the matrix product of the true 32-bit path (plain FMA, no reduced-precision
// tensor mode) and the one that takes every shape the tensor-core kernel refuses. It stands
// where the reference runs q8_gemv / q8_gemm_batched (src/cuda_resident.rs:230, :1494) with
// their fused residual add (:304-307). Each output element sums k = 0..K-1 in order, in
// chunks of 16, whatever M is and wherever the element lies in its tile: the value of a
// row does not depend on which other rows are in the batch.
//
// Epilogues: store in the input type; store float; add into a float matrix (the residual
// stream); SwiGLU, where output column j takes weight rows gate(j) and up(j) of a packed
// [2*N, K] matrix interleaved in groups of `group` rows and stores silu(g) * u.
#include "common.cuh"

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
    const float* a0p = A + (size_t)min(m0 + lrow0, M - 1) * lda + lkq;
    const float* a1p = A + (size_t)min(m0 + lrow1, M - 1) * lda + lkq;
    const float* w0p = W + (size_t)min(n0 + lrow0, n_wrows - 1) * ldw + lkq;
    const float* w1p = W + (size_t)min(n0 + lrow1, n_wrows - 1) * ldw + lkq;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

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
        Ws[buf][lkq + 0][lrow0] = rw0.x; Ws[buf][lkq + 1][lrow0] = rw0.y; Ws[buf][lkq + 2][lrow0] = rw0.z; Ws[buf][lkq + 3][lrow0] = rw0.w;
        Ws[buf][lkq + 0][lrow1] = rw1.x; Ws[buf][lkq + 1][lrow1] = rw1.y; Ws[buf][lkq + 2][lrow1] = rw1.z; Ws[buf][lkq + 3][lrow1] = rw1.w;
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
            const float4 bv0 = *reinterpret_cast<const float4*>(&Ws[buf][k][cg]);
            const float4 bv1 = *reinterpret_cast<const float4*>(&Ws[buf][k][cg + 16]);
            const float av[8] = {av0.x, av0.y, av0.z, av0.w, av1.x, av1.y, av1.z, av1.w};
            const float bv[8] = {bv0.x, bv0.y, bv0.z, bv0.w, bv1.x, bv1.y, bv1.z, bv1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
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
                    const float g = acc[i][j];
                    C[(size_t)r * ldc + c] = (g / (1.0f + expf(-g))) * acc[i][j + 4];
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
                    if (EPI == EPI_ADD_F32) *o += acc[i][4 * h + j];
                    else *o = acc[i][4 * h + j];
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

// Few rows in float, the form that streams weights: a block owns 32 consecutive weight rows and a
// range of K; its activations (MB rows of that range) are staged in shared memory once and every
// warp walks COLS weight rows at a time, so an activation read from shared memory serves COLS
// dot products and each lane keeps 2 * COLS 16-byte weight loads in flight. The first weight
// loads are issued before the wait on the previous kernel (weights do not depend on it). Where a
// product has too few 32-row tiles for the SMs, K is split over gridDim.y: every block leaves
// its sums in `scratch`, and the block that arrives last at the tile's ticket adds them in split
// order and runs the epilogue. The order of summation is fixed by N and K alone: lanes take
// their k's in ascending order, the lanes are summed in a fixed tree, the splits in index order.
// SwiGLU needs interleave groups of 16, so that a tile of 32 packed rows is 16 gate rows and the
// 16 up rows of the same outputs.
#define GV_WARPS 8
#define GV_ROWS 32          // weight rows per block
#define GV_AHEAD 2          // steps of 128 columns a lane has weight loads in flight for
template <int MB, int EPI>
__global__ void __launch_bounds__(GV_WARPS * 32, 2)
gemv_f32_stream_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw, float* __restrict__ C,
                       int ldc, int M, int n_wrows, int K, int kc, float* __restrict__ scratch, int* __restrict__ tickets) {
    constexpr int COLS = GV_ROWS / GV_WARPS;            // 4 weight rows per warp
    extern __shared__ __align__(16) float a_s[];        // [MB][kc]
    __shared__ int s_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tile = blockIdx.x, split = blockIdx.y, n_splits = gridDim.y;
    const int m0 = blockIdx.z * MB;
    const int k_begin = split * kc, k_end = min(K, k_begin + kc);
    const int steps = (k_end - k_begin + 127) / 128;
    const float* wp[COLS];
#pragma unroll
    for (int c = 0; c < COLS; ++c) wp[c] = W + (size_t)min(tile * GV_ROWS + warp * COLS + c, n_wrows - 1) * ldw;
    float acc[MB][COLS];
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int c = 0; c < COLS; ++c) acc[m][c] = 0.f;

    // weights of the first GV_AHEAD steps: on their way before the previous kernel has finished
    float4 w[GV_AHEAD][COLS];
#pragma unroll
    for (int u = 0; u < GV_AHEAD; ++u)
#pragma unroll
        for (int c = 0; c < COLS; ++c) w[u][c] = __ldg(reinterpret_cast<const float4*>(wp[c] + min(k_begin + u * 128 + lane * 4, K - 4)));
    pdl_wait();
    pdl_launch_dependents();
    for (int i = threadIdx.x; i < MB * (kc / 4); i += blockDim.x) {
        const int m = i / (kc / 4), k4 = (i - m * (kc / 4)) * 4;
        const int k = min(k_begin + k4, K - 4);
        *reinterpret_cast<float4*>(a_s + (size_t)m * kc + k4) =
            *reinterpret_cast<const float4*>(A + (size_t)min(m0 + m, M - 1) * lda + k);
    }
    __syncthreads();

    for (int st = 0; st < steps; st += GV_AHEAD) {
#pragma unroll
        for (int u = 0; u < GV_AHEAD; ++u) {
            const int kl = (st + u) * 128 + lane * 4;
            const bool live = k_begin + kl < k_end;      // past the range the clamped load does not count
            const int ka = min(kl, kc - 4);
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                const float4 a4 = live ? *reinterpret_cast<const float4*>(a_s + (size_t)m * kc + ka) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int c = 0; c < COLS; ++c) {
                    acc[m][c] = fmaf(a4.x, w[u][c].x, acc[m][c]); acc[m][c] = fmaf(a4.y, w[u][c].y, acc[m][c]);
                    acc[m][c] = fmaf(a4.z, w[u][c].z, acc[m][c]); acc[m][c] = fmaf(a4.w, w[u][c].w, acc[m][c]);
                }
            }
            // this slot's next weights, GV_AHEAD steps on (clamped to a valid address at the end)
            if (st + GV_AHEAD + u < steps) {
#pragma unroll
                for (int c = 0; c < COLS; ++c)
                    w[u][c] = __ldg(reinterpret_cast<const float4*>(wp[c] + min(k_begin + (st + GV_AHEAD + u) * 128 + lane * 4, K - 4)));
            }
        }
    }
    // this block's sums of its 32 weight rows, [MB][32], into shared memory (the staging area is free now)
    __syncthreads();
    float* sums = a_s;
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int c = 0; c < COLS; ++c) {
            const float v = warp_sum(acc[m][c]);
            if (lane == 0) sums[m * GV_ROWS + warp * COLS + c] = v;
        }
    __syncthreads();
    if (n_splits > 1) {
        float* mine = scratch + (((size_t)blockIdx.z * gridDim.x + tile) * n_splits + split) * (MB * GV_ROWS);
        for (int i = threadIdx.x; i < MB * GV_ROWS; i += blockDim.x) mine[i] = sums[i];
        __threadfence();
        __syncthreads();
        int* ticket = tickets + blockIdx.z * gridDim.x + tile;
        if (threadIdx.x == 0) {
            const int t = atomicAdd(ticket, 1);
            s_last = (t == n_splits - 1);
            if (s_last) *ticket = 0;                     // left zero for the next launch
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        const float* all = scratch + ((size_t)blockIdx.z * gridDim.x + tile) * n_splits * (MB * GV_ROWS);
        for (int i = threadIdx.x; i < MB * GV_ROWS; i += blockDim.x) {
            float v = 0.f;
            for (int sp = 0; sp < n_splits; ++sp) v += __ldcg(all + (size_t)sp * (MB * GV_ROWS) + i);
            sums[i] = v;
        }
        __syncthreads();
    }
    if (EPI == EPI_SWIGLU) {
        for (int i = threadIdx.x; i < MB * (GV_ROWS / 2); i += blockDim.x) {
            const int m = i / (GV_ROWS / 2), j = i - m * (GV_ROWS / 2);
            const int n = tile * (GV_ROWS / 2) + j;
            if (m0 + m < M && 2 * n < n_wrows) {
                const float g = sums[m * GV_ROWS + j], u = sums[m * GV_ROWS + GV_ROWS / 2 + j];
                C[(size_t)(m0 + m) * ldc + n] = (g / (1.0f + expf(-g))) * u;
            }
        }
    } else {
        for (int i = threadIdx.x; i < MB * GV_ROWS; i += blockDim.x) {
            const int m = i / GV_ROWS, j = i - m * GV_ROWS;
            const int n = tile * GV_ROWS + j;
            if (m0 + m < M && n < n_wrows) {
                float* o = C + (size_t)(m0 + m) * ldc + n;
                if (EPI == EPI_ADD_F32) *o += sums[i];
                else *o = sums[i];
            }
        }
    }
}

// Scratch the streaming form needs: tickets (ints, kept zero) in a first part of fixed size, which products of
// every shape share, then the splits' sums. K is split only where there are fewer than 3 * SMs tiles, and a
// step has at most 4 groups of 8 rows; a K beyond 2,048 columns is split whatever the tiles (an output head
// over a wide model). GV_TICKETS tickets cover half a million weight rows at four groups; more are refused.
#define GV_TICKETS 65536
static int gemv_stream_splits(int n_wrows, int K) {
    const int tiles = (n_wrows + GV_ROWS - 1) / GV_ROWS;
    int splits = (3 * cml_sm_count() + tiles - 1) / tiles;          // about three blocks per SM
    splits = max(1, min(splits, K / 512));                          // a range of at least 512 columns
    splits = max(splits, (K + 2047) / 2048);                        // and of at most 2,048 (shared memory)
    return splits;
}

extern "C" long cml_gemv_f32_scratch_bytes(int M, int N, int K, int epilogue) {
    const int n_wrows = epilogue == EPI_SWIGLU ? 2 * N : N;
    const int tiles = (n_wrows + GV_ROWS - 1) / GV_ROWS, groups = (M + 7) / 8;
    const int splits = gemv_stream_splits(n_wrows, K);
    return (long)GV_TICKETS * sizeof(int) + (splits > 1 ? (long)tiles * groups * splits * 8 * GV_ROWS * sizeof(float) : 0);
}

static int launch_gemv_f32_stream(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
                                  int epilogue, void* scratch, cudaStream_t s) {
    constexpr int MB = 8;
    const int n_wrows = epilogue == EPI_SWIGLU ? 2 * N : N;
    const int tiles = (n_wrows + GV_ROWS - 1) / GV_ROWS, groups = (M + MB - 1) / MB;
    const int splits = gemv_stream_splits(n_wrows, K);
    const int kc = ((K + splits - 1) / splits + 127) / 128 * 128;
    const int n_splits = (K + kc - 1) / kc;
    const size_t smem = (size_t)max(MB * kc, MB * GV_ROWS) * sizeof(float);
    if (n_splits > 1 && (long)tiles * groups > GV_TICKETS) return CML_ERR_BAD_SIZE;
    int* tickets = (int*)scratch;
    float* sums = (float*)((char*)scratch + (size_t)GV_TICKETS * sizeof(int));
    dim3 grid(tiles, n_splits, groups);
    cudaError_t e;
#define CML_GEMVS(E)                                                                                                   \
    e = cml_allow_smem<gemv_f32_stream_kernel<MB, E>>(smem);                                                           \
    if (e != cudaSuccess) return (int)e;                                                                               \
    launch_pdl(gemv_f32_stream_kernel<MB, E>, grid, dim3(GV_WARPS * 32), smem, s, (const float*)A, lda, (const float*)W, \
               ldw, (float*)C, ldc, M, n_wrows, K, kc, sums, tickets)
    switch (epilogue) {
        case EPI_STORE:
        case EPI_STORE_F32: CML_GEMVS(EPI_STORE_F32); break;
        case EPI_ADD_F32: CML_GEMVS(EPI_ADD_F32); break;
        case EPI_SWIGLU: CML_GEMVS(EPI_SWIGLU); break;
        default: return CML_ERR_BAD_SIZE;
    }
#undef CML_GEMVS
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
// first part (the tickets) is zero before the first call and left zero; with it, float products of at most 32 rows
// whose sizes allow 16-byte loads take the streaming form.
extern "C" int cml_gemm_tn_simt(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
                                int dtype, int epilogue, int group, void* scratch, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CML_DTYPE_F32 && M <= 32 && scratch != nullptr && K >= 128 && (K & 3) == 0 && (lda & 3) == 0 &&
        (ldw & 3) == 0 && (((uintptr_t)A | (uintptr_t)W) & 15) == 0 &&
        (epilogue != EPI_SWIGLU || (group == GV_ROWS / 2 && N % (GV_ROWS / 2) == 0)))
        return launch_gemv_f32_stream(A, lda, W, ldw, C, ldc, M, N, K, epilogue, scratch, s);
    if (dtype == CML_DTYPE_F32 && M <= 32) return launch_gemv_f32(A, lda, W, ldw, C, ldc, M, N, K, epilogue, group, s);
    if (dtype == CML_DTYPE_F32 && M >= 64 && (K & 3) == 0 && (lda & 3) == 0 && (ldw & 3) == 0 &&
        (((uintptr_t)A | (uintptr_t)W) & 15) == 0 && (epilogue != EPI_SWIGLU || (group == 16 && N % 16 == 0)))
        return launch_gemm_f32_big(A, lda, W, ldw, C, ldc, M, N, K, epilogue, s);
    if (dtype == CML_DTYPE_F32) return launch_gemm<float>(A, lda, W, ldw, C, ldc, M, N, K, epilogue, group, s);
    if (dtype == CML_DTYPE_BF16) return launch_gemm<bf16>(A, lda, W, ldw, C, ldc, M, N, K, epilogue, group, s);
    return CML_ERR_BAD_DTYPE;
}
