// Row-wise kernels: embedding gather, RMSNorm (optionally of gathered rows), SwiGLU on a
// packed gate/up matrix. One block per row; all arithmetic in float.
//
// What they replace in the reference: the host-side embedding_lookup
// (src/tensor/mod.rs:2253-2283) and embed_gather_* (src/cuda_resident.rs:2889-2995);
// rms_norm_f32 / rms_norm_batched (src/cuda_resident.rs:89, :1925), which sum with one
// thread to keep the CPU's order; silu_mul (src/cuda_resident.rs:1769).
#include "common.cuh"

// ------------------------------------------------------------------------------------
// out[r, :] = table[tokens[r], :]  (float residual stream). An id outside the vocabulary
// sets *err and writes zeros; the host checks ids before the launch, this is the net.
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                                    float* __restrict__ out, int hidden, int vocab, int* err) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int tok = tokens[r];
    float* o = out + (size_t)r * hidden;
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0) atomicOr(err, 1);
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[c] = 0.f;
        return;
    }
    const T* src = table + (size_t)tok * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[c] = to_f32(src[c]);
}

extern "C" int cml_embed_gather(const void* table, int dtype, const int* tokens, float* out, int rows,
                                int hidden, int vocab, int* err, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int block = hidden >= 1024 ? 256 : 128;
    if (dtype == CML_DTYPE_F32)
        launch_pdl(embed_gather_kernel<float>, dim3(rows), dim3(block), 0, s, (const float*)table, tokens, out, hidden, vocab, err);
    else if (dtype == CML_DTYPE_BF16)
        launch_pdl(embed_gather_kernel<bf16>, dim3(rows), dim3(block), 0, s, (const bf16*)table, tokens, out, hidden, vocab, err);
    else
        return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}

// ------------------------------------------------------------------------------------
// y = x * rsqrt(mean(x^2) + eps) * w, multiplied in that order (src/tensor/mod.rs:2086-2096).
// `rows_index` (may be null) picks the input row of each output row, so that the final norm
// runs only on the rows whose logits are wanted.
// `partial` (may be null) holds `n_splits` float matrices [x_rows, hidden] that are still to
// be added to x (the split sums of the product before): they are added in index order, and
// without `rows_index` the sum is written back to x, which settles the residual stream.
template <typename TW, typename TO>
__global__ void rmsnorm_kernel(float* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                               const int* __restrict__ rows_index, int hidden, float eps,
                               const float* __restrict__ partial, int n_splits, size_t split_stride) {
    __shared__ float red[33];
    extern __shared__ float rowbuf[];
    // the norm's weight does not depend on the kernels before: its first columns are fetched
    // ahead of the wait (each thread's first two columns cover hidden <= 2 * blockDim)
    const int c0 = threadIdx.x, c1 = threadIdx.x + blockDim.x;
    const float w0 = c0 < hidden ? to_f32(w[c0]) : 0.f;
    const float w1 = c1 < hidden ? to_f32(w[c1]) : 0.f;
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int src = rows_index ? rows_index[r] : r;
    float* xr = x + (size_t)src * hidden;
    float ss = 0.f;
    // Two columns of a thread at a time, and every load of both unconditional (of a valid
    // place, the value dropped where it does not count): all of them are in flight before the
    // first add. The adds stay in split order.
    for (int cb = threadIdx.x; cb < hidden; cb += 2 * blockDim.x) {
        const int cc[2] = {cb, cb + (int)blockDim.x};
        const bool in[2] = {true, cc[1] < hidden};
        float v[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) v[j] = xr[in[j] ? cc[j] : cb];
        if (partial) {
            for (int s0 = 0; s0 < n_splits; s0 += 8) {
                float t[2][8];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const float* pp = partial + (size_t)src * hidden + (in[j] ? cc[j] : cb);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float tv = pp[(size_t)min(s0 + i, n_splits - 1) * split_stride];
                        t[j][i] = (s0 + i < n_splits) ? tv : 0.f;
                    }
                }
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[j] += t[j][i];
            }
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            if (!in[j]) continue;
            if (partial) {
                rowbuf[cc[j]] = v[j];
                if (!rows_index) xr[cc[j]] = v[j];
            }
            ss = fmaf(v[j], v[j], ss);
        }
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
    TO* o = out + (size_t)r * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = partial ? rowbuf[c] : xr[c];
        const float wc = c == c0 ? w0 : (c == c1 ? w1 : to_f32(w[c]));
        o[c] = from_f32<TO>(v * scale * wc);
    }
}

// The same with split sums to add, when the row is a whole number of 16-byte groups: a thread
// owns groups of 4 columns, and the row's values and every split's reach it by cp.async into
// shared memory, all in flight at once (loads into registers, one chain of adds behind them,
// came out of the compiler as one round trip to L2 per few splits: 4 us of a 6 us launch). A
// thread reads back only what it copied itself, so no barrier stands between copy and use.
// Shared memory: the settled row [hidden], then [units_per_round][blockDim] groups.
template <typename TW, typename TO>
__global__ void rmsnorm_settle_kernel(float* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                                      const int* __restrict__ rows_index, int hidden, float eps,
                                      const float* __restrict__ partial, int n_splits, size_t split_stride,
                                      int units_per_round) {
    __shared__ float red[33];
    extern __shared__ __align__(16) float dyn[];
    float4* rowbuf = reinterpret_cast<float4*>(dyn);
    const float4* stage = reinterpret_cast<const float4*>(dyn + hidden);
    const uint32_t stage_u32 = (uint32_t)__cvta_generic_to_shared(dyn + hidden) + threadIdx.x * 16u;
    const int groups = hidden >> 2;
    const int g0 = threadIdx.x;
    float wv[4] = {0.f, 0.f, 0.f, 0.f};             // the norm's weight does not depend on the kernels before
    if (g0 < groups) {
#pragma unroll
        for (int i = 0; i < 4; ++i) wv[i] = to_f32(w[4 * g0 + i]);
    }
    const int r = blockIdx.x;
    const int units = n_splits + 1;                 // unit 0: the row itself; unit u: split u - 1
    if (!rows_index && g0 < groups) {
        // Touch what this thread will copy, ahead of the wait: the lines may still change (they
        // are only asked into L2, nothing is read), but the address translations are warm after.
        for (int u = 0; u < units; ++u) {
            const float* at = (u == 0) ? x + (size_t)r * hidden + 4 * g0 : partial + (size_t)(u - 1) * split_stride + (size_t)r * hidden + 4 * g0;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(at));
        }
    }
    pdl_wait();
    pdl_launch_dependents();
    const int src = rows_index ? rows_index[r] : r;
    float* xr = x + (size_t)src * hidden;
    const float* pr = partial + (size_t)src * hidden;
    float ss = 0.f;
    for (int g = threadIdx.x; g < groups; g += blockDim.x) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int u0 = 0; u0 < units; u0 += units_per_round) {
            const int nu = min(units_per_round, units - u0);
            for (int uu = 0; uu < nu; ++uu) {
                const float* from = (u0 + uu == 0) ? xr + 4 * g : pr + (size_t)(u0 + uu - 1) * split_stride + 4 * g;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(stage_u32 + (uint32_t)uu * blockDim.x * 16u), "l"(from) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            for (int uu = 0; uu < nu; ++uu) {       // the row, then the splits in order
                const float4 t = stage[(size_t)uu * blockDim.x + threadIdx.x];
                v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
            }
        }
        rowbuf[g] = v;
        if (!rows_index) *reinterpret_cast<float4*>(xr + 4 * g) = v;
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
    TO* o = out + (size_t)r * hidden;
    for (int g = threadIdx.x; g < groups; g += blockDim.x) {
        const float4 v = rowbuf[g];
        float wc[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) wc[i] = g == g0 ? wv[i] : to_f32(w[4 * g + i]);
        o[4 * g] = from_f32<TO>(v.x * scale * wc[0]);
        o[4 * g + 1] = from_f32<TO>(v.y * scale * wc[1]);
        o[4 * g + 2] = from_f32<TO>(v.z * scale * wc[2]);
        o[4 * g + 3] = from_f32<TO>(v.w * scale * wc[3]);
    }
}

template <typename TW, typename TO>
static int launch_rmsnorm_settle(float* x, const void* w, void* out, const int* rows_index, int rows, int hidden, float eps,
                                 const float* partial, int n_splits, long split_stride, cudaStream_t s) {
    const int groups = hidden / 4;
    int block = ((groups + 31) / 32) * 32;
    if (block > 1024) block = 1024;
    int upr = (96 * 1024) / (block * 16);
    if (upr > n_splits + 1) upr = n_splits + 1;
    if (upr < 1) upr = 1;
    const size_t smem = (size_t)hidden * sizeof(float) + (size_t)upr * block * 16;
    if (smem > 200 * 1024) return CML_ERR_BAD_SIZE;
    cudaError_t e = cml_allow_smem<rmsnorm_settle_kernel<TW, TO>>(smem);
    if (e != cudaSuccess) return (int)e;
    launch_pdl(rmsnorm_settle_kernel<TW, TO>, dim3(rows), dim3(block), smem, s, x, (const TW*)w, (TO*)out, rows_index, hidden,
               eps, partial, n_splits, (size_t)split_stride, upr);
    return cml_launch_status();
}

// Many rows (prefill): one warp per row, the row held in registers, so the row is read once
// and nothing waits on a block-wide barrier. VPL float4 per lane cover hidden = 128 * VPL.
template <typename TW, typename TO, int VPL>
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(const float* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                    const int* __restrict__ rows_index, int rows, int hidden, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31;
    const int src = rows_index ? rows_index[r] : r;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)src * hidden);
    float4 v[VPL];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int c = lane + 32 * i;                         // float4 index
        v[i] = (c * 4 < hidden) ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        ss = fmaf(v[i].x, v[i].x, ss);
        ss = fmaf(v[i].y, v[i].y, ss);
        ss = fmaf(v[i].z, v[i].z, ss);
        ss = fmaf(v[i].w, v[i].w, ss);
    }
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
    TO* o = out + (size_t)r * hidden;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int c = (lane + 32 * i) * 4;
        if (c >= hidden) continue;
        o[c] = from_f32<TO>(v[i].x * scale * to_f32(w[c]));
        o[c + 1] = from_f32<TO>(v[i].y * scale * to_f32(w[c + 1]));
        o[c + 2] = from_f32<TO>(v[i].z * scale * to_f32(w[c + 2]));
        o[c + 3] = from_f32<TO>(v[i].w * scale * to_f32(w[c + 3]));
    }
}

template <typename TW, typename TO>
static bool launch_rmsnorm_rows(const float* x, const void* w, void* out, const int* rows_index, int rows, int hidden,
                                float eps, cudaStream_t s) {
    if (hidden % 4 != 0 || hidden > 4096 || rows < 64) return false;
    const dim3 grid((rows + 7) / 8), block(256);
    const int vpl = (hidden / 4 + 31) / 32;
#define CML_ROWS(V) launch_pdl(rmsnorm_rows_kernel<TW, TO, V>, grid, block, 0, s, x, (const TW*)w, (TO*)out, rows_index, rows, hidden, eps)
    if (vpl <= 4) CML_ROWS(4);
    else if (vpl <= 8) CML_ROWS(8);
    else if (vpl <= 16) CML_ROWS(16);
    else if (vpl <= 32) CML_ROWS(32);
    else return false;
#undef CML_ROWS
    return true;
}

extern "C" int cml_rmsnorm(float* x, const void* w, int w_dtype, void* out, int out_dtype,
                           const int* rows_index, int rows, int hidden, float eps, const float* partial,
                           int n_splits, long split_stride, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (!partial) {
        bool done = false;
        if (w_dtype == CML_DTYPE_F32 && out_dtype == CML_DTYPE_F32) done = launch_rmsnorm_rows<float, float>(x, w, out, rows_index, rows, hidden, eps, s);
        else if (w_dtype == CML_DTYPE_F32 && out_dtype == CML_DTYPE_BF16) done = launch_rmsnorm_rows<float, bf16>(x, w, out, rows_index, rows, hidden, eps, s);
        else if (w_dtype == CML_DTYPE_BF16 && out_dtype == CML_DTYPE_F32) done = launch_rmsnorm_rows<bf16, float>(x, w, out, rows_index, rows, hidden, eps, s);
        else if (w_dtype == CML_DTYPE_BF16 && out_dtype == CML_DTYPE_BF16) done = launch_rmsnorm_rows<bf16, bf16>(x, w, out, rows_index, rows, hidden, eps, s);
        if (done) return cml_launch_status();
    }
    if (partial && hidden % 4 == 0 && split_stride % 4 == 0 && (((uintptr_t)x | (uintptr_t)partial) & 15) == 0 &&
        (size_t)hidden * sizeof(float) <= 100 * 1024) {
        if (w_dtype == CML_DTYPE_F32 && out_dtype == CML_DTYPE_F32) return launch_rmsnorm_settle<float, float>(x, w, out, rows_index, rows, hidden, eps, partial, n_splits, split_stride, s);
        if (w_dtype == CML_DTYPE_F32 && out_dtype == CML_DTYPE_BF16) return launch_rmsnorm_settle<float, bf16>(x, w, out, rows_index, rows, hidden, eps, partial, n_splits, split_stride, s);
        if (w_dtype == CML_DTYPE_BF16 && out_dtype == CML_DTYPE_F32) return launch_rmsnorm_settle<bf16, float>(x, w, out, rows_index, rows, hidden, eps, partial, n_splits, split_stride, s);
        if (w_dtype == CML_DTYPE_BF16 && out_dtype == CML_DTYPE_BF16) return launch_rmsnorm_settle<bf16, bf16>(x, w, out, rows_index, rows, hidden, eps, partial, n_splits, split_stride, s);
        return CML_ERR_BAD_DTYPE;
    }
    // few rows (decode): many threads per row shorten the chain; many rows: several blocks per SM
    const int block = hidden >= 1024 ? (rows <= 256 ? 1024 : 256) : (hidden >= 512 ? 256 : 128);
    const size_t smem = partial ? (size_t)hidden * sizeof(float) : 0;
    if (smem > 48 * 1024) return CML_ERR_BAD_SIZE;
#define CML_RMS(TW, TO) launch_pdl(rmsnorm_kernel<TW, TO>, dim3(rows), dim3(block), smem, s, x, (const TW*)w, (TO*)out, rows_index, hidden, eps, partial, n_splits, (size_t)split_stride)
    if (w_dtype == CML_DTYPE_F32 && out_dtype == CML_DTYPE_F32) CML_RMS(float, float);
    else if (w_dtype == CML_DTYPE_F32 && out_dtype == CML_DTYPE_BF16) CML_RMS(float, bf16);
    else if (w_dtype == CML_DTYPE_BF16 && out_dtype == CML_DTYPE_F32) CML_RMS(bf16, float);
    else if (w_dtype == CML_DTYPE_BF16 && out_dtype == CML_DTYPE_BF16) CML_RMS(bf16, bf16);
    else return CML_ERR_BAD_DTYPE;
#undef CML_RMS
    return cml_launch_status();
}

// ------------------------------------------------------------------------------------
// act[r, j] = silu(g) * u with g / (1 + exp(-g)) (src/inference.rs:9657-9664), on a packed
// matrix gu[r, 2*inter] whose rows of weights were interleaved in groups of `group`:
// gate j sits at column (j / group) * 2 * group + j % group, up j `group` columns later.
template <typename T>
__global__ void swiglu_packed_kernel(const T* __restrict__ gu, T* __restrict__ act, int inter, int group) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const T* row = gu + (size_t)r * 2 * inter;
    T* o = act + (size_t)r * inter;
    for (int j = threadIdx.x; j < inter; j += blockDim.x) {
        const int col = (j / group) * 2 * group + j % group;
        const float g = to_f32(row[col]);
        const float u = to_f32(row[col + group]);
        o[j] = from_f32<T>((g / (1.0f + expf(-g))) * u);
    }
}

extern "C" int cml_swiglu_packed(const void* gu, void* act, int dtype, int rows, int inter, int group, void* stream) {
    if (rows <= 0) return 0;
    if (group <= 0 || inter % group != 0) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CML_DTYPE_F32)
        launch_pdl(swiglu_packed_kernel<float>, dim3(rows), dim3(256), 0, s, (const float*)gu, (float*)act, inter, group);
    else if (dtype == CML_DTYPE_BF16)
        launch_pdl(swiglu_packed_kernel<bf16>, dim3(rows), dim3(256), 0, s, (const bf16*)gu, (bf16*)act, inter, group);
    else
        return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}

// ------------------------------------------------------------------------------------
// x += sum_s partial[s] (float), splits in index order: settles split sums that no norm
// kernel picked up.
__global__ void add_partials_kernel(float* __restrict__ x, const float* __restrict__ partial, int n_splits, long n) {
    pdl_wait();
    pdl_launch_dependents();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = x[i];
    for (int s = 0; s < n_splits; ++s) v += partial[(size_t)s * n + i];
    x[i] = v;
}

extern "C" int cml_add_partials(float* x, const float* partial, int n_splits, long n, void* stream) {
    if (n <= 0 || n_splits <= 0) return 0;
    launch_pdl(add_partials_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, x, partial, n_splits, n);
    return cml_launch_status();
}

// x[r][:] *= rsqrt(sum_t sumsq[t][r] / hidden + eps): gives rows that came out of a norm without
// their scale (see cml_gemm_tc_pair_add_norm) that scale, for a consumer that cannot apply it.
template <typename T>
__global__ void scale_rows_kernel(T* __restrict__ x, long ldx, int width, const float* __restrict__ sumsq, int parts,
                                  int rows, float inv_hidden, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    float ssq = 0.f;
    for (int t = 0; t < parts; ++t) ssq += sumsq[(size_t)t * rows + r];
    const float scale = 1.0f / sqrtf(ssq * inv_hidden + eps);
    T* row = x + (size_t)r * ldx;
    for (int c = threadIdx.x; c < width; c += blockDim.x) row[c] = from_f32<T>(to_f32(row[c]) * scale);
}

extern "C" int cml_scale_rows(void* x, int dtype, long ldx, int rows, int width, const float* sumsq, int parts, int hidden,
                              float eps, void* stream) {
    if (rows <= 0 || width <= 0) return 0;
    if (parts < 1 || hidden < 1) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CML_DTYPE_F32)
        launch_pdl(scale_rows_kernel<float>, dim3(rows), dim3(256), 0, s, (float*)x, ldx, width, sumsq, parts, rows, 1.0f / (float)hidden, eps);
    else if (dtype == CML_DTYPE_BF16)
        launch_pdl(scale_rows_kernel<bf16>, dim3(rows), dim3(256), 0, s, (bf16*)x, ldx, width, sumsq, parts, rows, 1.0f / (float)hidden, eps);
    else
        return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}
