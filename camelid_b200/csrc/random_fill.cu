// Random weights on the device: element i of a tensor with key `key` is
//     float32(mean + std * sqrt(-2 ln u1) * cos(angle)),
// u1 and the angle being the two halves of splitmix64(key + (i + 1) * golden). The host
// twin (weights/counter_random.py) runs the same arithmetic step by step, and both use only
// operations that IEEE 754 rounds correctly, so the two agree bit for bit: every product,
// sum, quotient and root below is an explicitly rounded intrinsic, which the compiler never
// contracts into a fused multiply-add.
//
// The reference draws random weights only in its tests, with a linear congruential
// generator on the host (src/cuda_resident/tests.rs:537-553).
#include "common.cuh"

namespace {

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ double mul(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ double add(double a, double b) { return __dadd_rn(a, b); }

// 1 / (2k + 1), (-1)^k / (2k)!, (-1)^k / (2k + 1)!: quotients of exactly representable
// numbers, folded by the compiler with the same correct rounding as the host's division.
__constant__ double LOG_TERMS[11] = {1.0, 1.0 / 3.0, 1.0 / 5.0, 1.0 / 7.0, 1.0 / 9.0, 1.0 / 11.0, 1.0 / 13.0,
                                     1.0 / 15.0, 1.0 / 17.0, 1.0 / 19.0, 1.0 / 21.0};
__constant__ double COS_TERMS[9] = {1.0, -1.0 / 2.0, 1.0 / 24.0, -1.0 / 720.0, 1.0 / 40320.0, -1.0 / 3628800.0,
                                    1.0 / 479001600.0, -1.0 / 87178291200.0, 1.0 / 20922789888000.0};
__constant__ double SIN_TERMS[9] = {1.0, -1.0 / 6.0, 1.0 / 120.0, -1.0 / 5040.0, 1.0 / 362880.0, -1.0 / 39916800.0,
                                    1.0 / 6227020800.0, -1.0 / 1307674368000.0, 1.0 / 355687428096000.0};

template <int N>
__device__ __forceinline__ double horner(const double* terms, double w) {
    double p = terms[N - 1];
#pragma unroll
    for (int k = N - 2; k >= 0; --k) p = add(mul(p, w), terms[k]);
    return p;
}

__device__ __forceinline__ double standard_normal(unsigned long long key, unsigned long long i) {
    const unsigned long long z = splitmix64(key + (i + 1ull) * 0x9E3779B97F4A7C15ull);
    const double n = add((double)(unsigned int)(z >> 32), 1.0);          // 1 .. 2^32, exact
    const unsigned int b = (unsigned int)z;
    int ex;
    double mant = frexp(n, &ex);                                         // n = mant * 2^ex, mant in [0.5, 1)
    if (mant < 0.7071067811865476) { mant = mul(mant, 2.0); ex -= 1; }
    const double s = __ddiv_rn(add(mant, -1.0), add(mant, 1.0));
    const double ln_u = add(mul((double)(ex - 32), 0.6931471805599453), mul(mul(2.0, s), horner<11>(LOG_TERMS, mul(s, s))));
    const double r = __dsqrt_rn(mul(-2.0, ln_u));
    const unsigned int octant = b >> 29;
    const double f = mul((double)(b & 0x1FFFFFFFu), 1.0 / 536870912.0);
    const double g = (octant & 1u) ? add(1.0, -f) : f;
    const double t = mul(g, 0.7853981633974483);
    const double w = mul(t, t);
    const bool use_sin = ((octant + 1u) & 2u) != 0;                      // octants 1, 2, 5, 6
    const bool negative = ((octant + 2u) & 4u) != 0;                     // octants 2, 3, 4, 5
    double trig = use_sin ? mul(t, horner<9>(SIN_TERMS, w)) : horner<9>(COS_TERMS, w);
    if (negative) trig = -trig;
    return mul(r, trig);
}

template <typename T>
__global__ void random_fill_kernel(T* __restrict__ out, size_t count, unsigned long long key, unsigned long long first,
                                   double mean, double std) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        const float v = __double2float_rn(add(mean, mul(std, standard_normal(key, first + i))));
        out[i] = from_f32<T>(v);
    }
}

}  // namespace

// out[i] = value of element first + i, i < count; float32 or (rounded from the float32 value) bfloat16.
extern "C" int cml_random_fill(void* out, int dtype, long long count, unsigned long long key, unsigned long long first,
                               double mean, double std, void* stream) {
    if (count <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int block = 256;
    long long want = (count + block - 1) / block;
    const int grid = (int)(want < (long long)cml_sm_count() * 16 ? want : (long long)cml_sm_count() * 16);
    if (dtype == CML_DTYPE_F32)
        random_fill_kernel<float><<<grid, block, 0, s>>>((float*)out, (size_t)count, key, first, mean, std);
    else if (dtype == CML_DTYPE_BF16)
        random_fill_kernel<bf16><<<grid, block, 0, s>>>((bf16*)out, (size_t)count, key, first, mean, std);
    else
        return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}
