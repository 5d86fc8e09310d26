// Sampling on the device: greedy argmax and the reference's stochastic sampler
// (temperature, top-k, min-p, top-p), a cluster of up to eight blocks per row of logits.
//
// Greedy follows greedy_sample (src/inference.rs:5890-5925; device twin argmax_f32 at
// src/cuda_resident.rs:1847): strict '>', so the lowest index among equal maxima wins, and
// non-finite logits are an error. The stochastic sampler follows sample_with_config
// (src/inference.rs:5991-6091): candidates ordered by logit descending with ties by index
// ascending; top_k keeps a prefix; softmax of logit/T minus its maximum; min_p keeps
// p >= min_p * p_max and renormalises; top_p keeps the shortest prefix whose cumulative
// probability reaches top_p and renormalises; the token is the first whose cumulative
// probability exceeds the draw. The reference sorts; here every stage is a selection in the
// same total order: in two passes over the row where that settles it (bins of the distance
// from the maximum locate the crossing, the one bin's keys are sorted and walked), else by
// descending the bits of a 64-bit key (orderable logit bits, then inverted index) with
// per-digit histograms of weight. Sums are
// kept in double; the reference's sequential float sums can differ from them in the last
// bits, which moves a decision only when the draw or top_p lies on a boundary.
#include "common.cuh"
#include <cooperative_groups.h>
#include <math_constants.h>
namespace cg = cooperative_groups;

#define SAMPLE_THREADS 1024
#define SAMPLE_MAX_TEAM 8      // blocks that may share a row (a portable cluster)
#define SAMPLE_LIST_WALK 512    // a top_k up to this is finished along its sorted list by one thread
#define SAMPLE_ERR_NONFINITE 1
#define SAMPLE_ERR_EMPTY 2

__device__ __forceinline__ unsigned int orderable_bits(float v) {
    const unsigned int u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);       // larger float -> larger unsigned
}
__device__ __forceinline__ unsigned long long composite_key(float v, int idx) {
    return ((unsigned long long)orderable_bits(v) << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned int)idx);
}

// ------------------------------------------------------------------------------------
// Greedy choice per row, spread over several blocks per row so that a large vocabulary is
// read at memory speed. Every block folds its part into one 64-bit word per row with
// atomicMax: the orderable bits of the logit above, the inverted index below, so that the
// largest logit wins and among equals the lowest index. The block that arrives last (a
// counter per row) writes the token and clears the row's two words for the next call.
// `scratch` holds 2 * rows unsigned 64-bit words, zero before the first call.
__global__ void argmax_rows_kernel(const float* __restrict__ logits, int ld, int vocab, int* __restrict__ out,
                                   int* __restrict__ err, unsigned long long* __restrict__ scratch) {
    __shared__ unsigned long long red[32];
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.y;
    const float* r = logits + (size_t)row * ld;
    // parts of whole groups of four columns, so that aligned rows are read 16 bytes at a time
    const int per = ((vocab + gridDim.x - 1) / gridDim.x + 3) & ~3;
    const int begin = min(vocab, blockIdx.x * per), end = min(vocab, begin + per);
    // A thread walks its columns in ascending order, so "strictly larger" keeps the lowest index among equals;
    // the 64-bit word is made once, at the end.
    float bv = -CUDART_INF_F;
    int bi = -1;
    bool bad = false;
    auto take = [&](float v, int i) {
        bad = bad || !(fabsf(v) < CUDART_INF_F);              // infinite or not a number
        if (v > bv || bi < 0) {
            bv = v;
            bi = i;
        }
    };
    if ((((uintptr_t)r) & 15) == 0) {
        const int end4 = begin + ((end - begin) & ~3);
        // four loads of 16 bytes in flight per thread (unconditional, of a clamped place), then their values
        for (int i0 = begin + 4 * threadIdx.x; i0 < end4; i0 += 16 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const float4*>(r + min(i0 + u * 4 * (int)blockDim.x, end4 - 4));
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * 4 * (int)blockDim.x;
                if (i < end4) {
                    take(v[u].x, i); take(v[u].y, i + 1); take(v[u].z, i + 2); take(v[u].w, i + 3);
                }
            }
        }
        for (int i = end4 + threadIdx.x; i < end; i += blockDim.x) take(r[i], i);
    } else {
        for (int i = begin + threadIdx.x; i < end; i += blockDim.x) take(r[i], i);
    }
    if (bad) atomicOr(err, SAMPLE_ERR_NONFINITE);
    unsigned long long best = bi >= 0 ? composite_key(bv + 0.0f, bi) : 0ull;      // -0 as +0: equal, the lower index wins
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if (lane == 0) red[warp] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) best = red[w] > best ? red[w] : best;
        unsigned long long* cell = scratch + 2 * (size_t)row;
        if (best) atomicMax(cell, best);
        __threadfence();
        const unsigned long long ticket = atomicAdd(cell + 1, 1ull);
        if (ticket == gridDim.x - 1) {
            __threadfence();
            const unsigned long long win = atomicExch(cell, 0ull);
            out[row] = win ? (int)(0xFFFFFFFFu - (unsigned int)(win & 0xFFFFFFFFull)) : 0;
            cell[1] = 0ull;
        }
    }
}

// Blocks per row: enough for two a multiprocessor over all rows and for at most two rounds of four 16-byte loads
// a thread (8,192 columns a block), none with less than 2,048 columns.
static int argmax_blocks(int rows, int vocab) {
    return max(1, min(min(64, vocab / 2048), max((2 * cml_sm_count() + rows - 1) / rows, (vocab + 8191) / 8192)));
}

extern "C" int cml_argmax_rows(const float* logits, int ld, int rows, int vocab, int* out, int* err,
                               unsigned long long* scratch, void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || rows > 65535) return CML_ERR_BAD_SIZE;
    const int blocks = argmax_blocks(rows, vocab);
    launch_pdl(argmax_rows_kernel, dim3(blocks, rows), dim3(256), 0, (cudaStream_t)stream, logits, ld, vocab, out, err, scratch);
    return cml_launch_status();
}

// ------------------------------------------------------------------------------------
// Adjustments before sampling (src/inference.rs:6093-6157): for each listed (row, token,
// count, bias) entry, logit += bias; then, if count > 0: repeat penalty (divide a positive
// logit, multiply a negative one), minus presence, minus frequency * count. The host builds
// the list from the history (one entry per distinct token) and the bias table.
__global__ void adjust_logits_kernel(float* __restrict__ logits, int ld, int vocab, const int* __restrict__ entries,
                                     const float* __restrict__ biases, int n_entries, float repeat_penalty,
                                     float presence_penalty, float frequency_penalty) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n_entries) return;
    const int row = entries[3 * e], tok = entries[3 * e + 1], count = entries[3 * e + 2];
    if (tok < 0 || tok >= vocab) return;
    float v = logits[(size_t)row * ld + tok] + biases[e];
    if (count > 0) {
        if (repeat_penalty != 1.0f) v = v > 0.f ? v / repeat_penalty : v * repeat_penalty;
        if (presence_penalty != 0.0f) v -= presence_penalty;
        if (frequency_penalty != 0.0f) v -= frequency_penalty * (float)count;
    }
    logits[(size_t)row * ld + tok] = v;
}

extern "C" int cml_adjust_logits(float* logits, int ld, int vocab, const int* entries, const float* biases,
                                 int n_entries, float repeat_penalty, float presence_penalty,
                                 float frequency_penalty, void* stream) {
    if (n_entries <= 0) return 0;
    adjust_logits_kernel<<<(n_entries + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
        logits, ld, vocab, entries, biases, n_entries, repeat_penalty, presence_penalty, frequency_penalty);
    return cml_launch_status();
}

// The same adjustments from counts kept on the device, for steps that feed themselves: counts[r][t] is how often
// token t stands in row r's history, bias[t] the sum of the biases listed for t (0 elsewhere: adding it changes
// nothing), penalties = {repeat, presence, frequency} in device memory, so that one captured graph serves any
// values. count_tokens adds the tokens a step has chosen to their rows' counts.
__global__ void adjust_dense_kernel(float* __restrict__ logits, int ld, int vocab, const int* __restrict__ counts,
                                    const float* __restrict__ bias, const float* __restrict__ penalties) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y;
    if (t >= vocab) return;
    const float repeat_penalty = penalties[0], presence_penalty = penalties[1], frequency_penalty = penalties[2];
    const int count = counts[(size_t)row * vocab + t];
    const float b = bias[t];
    if (count == 0 && b == 0.f) return;
    float v = logits[(size_t)row * ld + t] + b;
    if (count > 0) {
        if (repeat_penalty != 1.0f) v = v > 0.f ? v / repeat_penalty : v * repeat_penalty;
        if (presence_penalty != 0.0f) v -= presence_penalty;
        if (frequency_penalty != 0.0f) v -= frequency_penalty * (float)count;
    }
    logits[(size_t)row * ld + t] = v;
}

__global__ void count_tokens_kernel(const int* __restrict__ tokens, int* __restrict__ counts, int rows, int vocab) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const int t = tokens[r];
    if (t >= 0 && t < vocab) counts[(size_t)r * vocab + t] += 1;
}

extern "C" int cml_adjust_dense(float* logits, int ld, int rows, int vocab, const int* counts, const float* bias,
                                const float* penalties, void* stream) {
    if (rows <= 0 || vocab <= 0) return 0;
    if (rows > 65535) return CML_ERR_BAD_SIZE;
    adjust_dense_kernel<<<dim3((vocab + 255) / 256, rows), 256, 0, (cudaStream_t)stream>>>(logits, ld, vocab, counts, bias,
                                                                                          penalties);
    return cml_launch_status();
}

extern "C" int cml_count_tokens(const int* tokens, int* counts, int rows, int vocab, void* stream) {
    if (rows <= 0) return 0;
    count_tokens_kernel<<<(rows + 127) / 128, 128, 0, (cudaStream_t)stream>>>(tokens, counts, rows, vocab);
    return cml_launch_status();
}

// ------------------------------------------------------------------------------------
// Selection in the total order (key descending). The weight of element i is given by the
// functor; elements with key < floor_key are not candidates. Finds the first candidate at
// which the inclusive cumulative weight reaches (`strict` 0: >=, 1: >) the target, and
// returns its key and that inclusive sum. If the total never reaches the target the last
// candidate (floor) is returned with the total.
struct SelectShared {
    double mass[256];
    unsigned int count[256];
    unsigned long long prefix;
    double before;
    int chosen;
    int found;
};

template <typename WeightFn>
__device__ void select_by_mass(const float* row, int vocab, unsigned long long floor_key, double target, int strict,
                               WeightFn weight, SelectShared* sh, unsigned long long* out_key, double* out_cum) {
    unsigned long long prefix = 0;      // digits chosen so far, in place
    double before = 0.0;                // mass of candidates ordered before the chosen prefix
    for (int shift = 56; shift >= 0; shift -= 8) {
        for (int b = threadIdx.x; b < 256; b += blockDim.x) sh->mass[b] = 0.0, sh->count[b] = 0u;
        __syncthreads();
        const unsigned long long hi_mask = shift == 56 ? 0ull : (~0ull << (shift + 8));
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float v = row[i];
            const unsigned long long key = composite_key(v, i);
            if (key < floor_key || (key & hi_mask) != prefix) continue;
            const int bin = (int)((key >> shift) & 0xFFull);
            atomicAdd(&sh->mass[bin], (double)weight(v, i));
            atomicAdd(&sh->count[bin], 1u);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            double acc = before;
            int chosen = -1, last = -1;
            for (int b = 255; b >= 0; --b) {
                if (sh->count[b] == 0u) continue;
                last = b;
                const double inc = acc + sh->mass[b];
                if (strict ? (inc > target) : (inc >= target)) { chosen = b; break; }
                acc = inc;
            }
            if (chosen < 0) {           // never reached: settle on the last candidate
                chosen = last;
                acc -= sh->mass[last];
            }
            sh->chosen = chosen;
            sh->before = acc;
        }
        __syncthreads();
        if (sh->chosen < 0) {           // no candidate at all
            *out_key = floor_key;
            *out_cum = before;
            return;
        }
        prefix |= ((unsigned long long)sh->chosen) << shift;
        before = sh->before;
        __syncthreads();
    }
    // prefix is now the full key of one element
    if (threadIdx.x == 0) sh->found = 0;
    __syncthreads();
    *out_key = prefix;
    const int idx = (int)(0xFFFFFFFFu - (unsigned int)(prefix & 0xFFFFFFFFull));
    double w = 0.0;
    if (idx >= 0 && idx < vocab) w = (double)weight(row[idx], idx);
    *out_cum = before + w;
}

// The blocks that share a row of logits: a thread-block cluster (of one block where the row is short). Every
// block scans its own slice of the row; what they find meets in the shared memory of block 0 (distributed shared
// memory), between cluster barriers.
struct Team {
    int n, rank;
    int begin, end;              // this block's slice of the row (begin a multiple of 4)
    __device__ void sync() { cg::this_cluster().sync(); }
    template <typename T> __device__ T* at0(T* p) { return cg::this_cluster().map_shared_rank(p, 0); }
};

// What a reduction over the team passes through block 0: one slot per block and place of use, written before a
// cluster barrier and read after it by whoever needs the result (every block, or block 0 alone).
struct TeamSlots {
    double d[4][SAMPLE_MAX_TEAM];
    float f[2][SAMPLE_MAX_TEAM];
    unsigned int u[2][SAMPLE_MAX_TEAM];
    unsigned long long k[1][SAMPLE_MAX_TEAM];
};

// Every element of this block's slice to `f(value, index)`, a thread's elements in ascending index order. Rows
// that start on a 16-byte boundary are read 16 bytes at a time, two such loads in flight per thread (a scan with
// one 4-byte load at a time is bound by the loads' round trips).
template <typename F>
__device__ __forceinline__ void for_each_in_slice(const float* __restrict__ row, const Team& tm, F f) {
    const int begin = tm.begin, end = tm.end;
    if ((((uintptr_t)row) & 15) == 0) {
        const int g_begin = begin >> 2, g_end = end >> 2;          // whole groups of four within the slice
        const float4* r4 = reinterpret_cast<const float4*>(row);
        for (int g0 = g_begin + threadIdx.x; g0 < g_end; g0 += 2 * blockDim.x) {
            const int g1 = g0 + blockDim.x;
            const float4 a = r4[g0];
            const float4 b = r4[min(g1, g_end - 1)];
            f(a.x, 4 * g0); f(a.y, 4 * g0 + 1); f(a.z, 4 * g0 + 2); f(a.w, 4 * g0 + 3);
            if (g1 < g_end) { f(b.x, 4 * g1); f(b.y, 4 * g1 + 1); f(b.z, 4 * g1 + 2); f(b.w, 4 * g1 + 3); }
        }
        for (int i = max(begin, 4 * g_end) + threadIdx.x; i < end; i += blockDim.x) f(row[i], i);
    } else {
        for (int i = begin + threadIdx.x; i < end; i += blockDim.x) f(row[i], i);
    }
}

// Maximum over the block, in every thread. `scratch33`: 33 floats of shared memory.
__device__ __forceinline__ float block_max(float v, float* scratch33) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch33[warp] = v;
    __syncthreads();
    return warp_max(lane < nw ? scratch33[lane] : -CUDART_INF_F);
}

// Sum over the block; the result is valid in thread 0.
__device__ __forceinline__ double block_sum_double(double v, double* scratch33) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch33[warp] = v;
    __syncthreads();
    double t = 0.0;
    if (threadIdx.x == 0)
        for (int w = 0; w < nw; ++w) t += scratch33[w];
    return t;
}

// ------------------------------------------------------------------------------------
// The same selection in two passes over the row instead of eight, for the usual case. The order of the
// candidates is by value descending, so by x = max / T - value / T ascending. A first pass counts the
// candidates and adds their weights (in float: only to find the place) into 2,048 bins of x; the bin in which
// the cumulative weight reaches the target is found from those. A second pass adds, in double, the weights of
// all candidates ordered before that bin and collects the bin's own keys, which are then sorted and walked
// exactly as the selection above walks them. If the exact sums put the crossing into a neighbouring bin, that
// bin is taken and the second pass repeated. A bin with more keys than the list holds is divided into 2,048
// bins of its own (twice at most: then its keys are equal values, and the selection above, which orders equal
// values by index digit by digit, takes over).
#define FS_BINS 2048
#define FS_CAP 2048
struct FastShared {
    unsigned int cnt[FS_BINS];
    float mass[FS_BINS];
    unsigned long long list[FS_CAP];
    float lp[FS_CAP];
    double dred[33];
    unsigned int n_list;
    int bin;
    int status;              // 0: walk again with `bin`; 1: found; 2: divide the bin; 3: give up (fall back)
    unsigned long long key;
    double cum;
};

__device__ __forceinline__ float value_of_key(unsigned long long key) {
    const unsigned int u = (unsigned int)(key >> 32);
    return __uint_as_float((u & 0x80000000u) ? (u & 0x7FFFFFFFu) : ~u);
}

// Returns true and the choice if the fast way settled it, false if the caller has to run select_by_mass.
// `xof(v)` is the place of a value in the order (smaller first, monotone in v), `weight(v, i)` as above,
// `approx(x)` a cheap estimate of the weight of a value at place x, good enough to find the bin.
template <typename XFn, typename WeightFn, typename ApproxFn>
__device__ bool select_fast(const float* row, Team& tm, unsigned long long floor_key, double target, int strict,
                            XFn xof, float x_max, WeightFn weight, ApproxFn approx, FastShared* fs, TeamSlots* ts,
                            unsigned long long* out_key, double* out_cum) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    FastShared* fs0 = tm.at0(fs);                        // block 0's: the merged bins, the list, the verdicts
    TeamSlots* ts0 = tm.at0(ts);
    float lo = 0.f, inv_w = 64.0f;                       // bins of 1/64 from 0; the last one takes all beyond
    bool open_end = true;
    for (int level = 0; level < 3; ++level) {
        // pass 1: counts and approximate weights of the candidates per bin of [lo, ...), block by block
        for (int b = threadIdx.x; b < FS_BINS; b += blockDim.x) fs->cnt[b] = 0u, fs->mass[b] = 0.f;
        tm.sync();                                       // block 0's bins are clear before anyone adds to them
        auto bin_at = [&](float x) {                     // -1: ordered before the range; FS_BINS: after it
            const float r = (x - lo) * inv_w;
            if (r < 0.f) return -1;
            if (r >= (float)FS_BINS) return open_end ? FS_BINS - 1 : FS_BINS;
            return (int)r;
        };
        auto bin_of = [&](float v) { return bin_at(xof(v)); };
        const bool has_floor = floor_key != 0ull;
        double head = 0.0;                               // weight ordered before the range
        for_each_in_slice(row, tm, [&](float v, int i) {
            if (has_floor && composite_key(v, i) < floor_key) return;
            const float x = xof(v);
            const int b = bin_at(x);
            if (b < 0) head += (double)weight(v, i);
            else if (b < FS_BINS) {
                atomicAdd(&fs->cnt[b], 1u);
                atomicAdd(&fs->mass[b], approx(x));
            }
        });
        head = block_sum_double(head, fs->dred);
        if (threadIdx.x == 0) ts0->d[0][tm.rank] = head;
        if (tm.rank != 0) {                              // this block's bins into block 0's
            for (int b = threadIdx.x; b < FS_BINS; b += blockDim.x) {
                const unsigned int c = fs->cnt[b];
                if (c != 0u) {
                    atomicAdd(&fs0->cnt[b], c);
                    atomicAdd(&fs0->mass[b], fs->mass[b]);
                }
            }
        }
        tm.sync();
        if (tm.rank == 0 && warp == 0) {
            // a lane sums 64 consecutive bins; the lane in which the cumulative weight reaches the target walks its own
            double acc0 = 0.0;
            for (int r = 0; r < tm.n; ++r) acc0 += ts->d[0][r];
            constexpr int PER = FS_BINS / 32;
            double mine = 0.0;
            int my_last = -1;
            for (int b = lane * PER; b < (lane + 1) * PER; ++b) {
                if (fs->cnt[b] == 0u) continue;
                my_last = b;
                mine += (double)fs->mass[b];
            }
            double incl = mine;                          // inclusive sum over lanes
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            const double upto = acc0 + incl;             // weight up to the end of this lane's bins
            const bool reach = my_last >= 0 && (strict ? (upto > target) : (upto >= target));
            const unsigned int who = __ballot_sync(0xffffffffu, reach);
            int last = my_last;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) last = max(last, __shfl_xor_sync(0xffffffffu, last, o));
            if (who != 0u && lane == __ffs(who) - 1) {
                double acc = upto - mine;
                int chosen = -1;
                for (int b = lane * PER; b < (lane + 1) * PER; ++b) {
                    if (fs->cnt[b] == 0u) continue;
                    const double inc = acc + (double)fs->mass[b];
                    if (strict ? (inc > target) : (inc >= target)) { chosen = b; break; }
                    acc = inc;
                }
                if (chosen < 0) chosen = my_last;        // rounding between the two sums: the lane's last bin
                fs->bin = chosen;
                fs->status = 0;
            }
            if (who == 0u && lane == 0) {
                fs->bin = last;                          // never reached: the last bin with candidates
                fs->status = last < 0 ? 3 : 0;           // no candidate in the range at all: not ours
            }
            if (lane == 0) fs->n_list = 0u;
        }
        tm.sync();
        if (fs0->status == 3) { tm.sync(); return false; }
        // pass 2, repeated while the exact sums move the crossing to a neighbouring bin
        int st = 0;
        for (int tries = 0; tries < 6; ++tries) {
            const int bsel = fs0->bin;
            double before = 0.0;
            unsigned int after = 0u;
            for_each_in_slice(row, tm, [&](float v, int i) {
                if (has_floor && composite_key(v, i) < floor_key) return;
                const int b = bin_of(v);
                if (b < bsel) before += (double)weight(v, i);
                else if (b == bsel) {
                    const unsigned int slot = atomicAdd(&fs0->n_list, 1u);
                    if (slot < FS_CAP) fs0->list[slot] = composite_key(v, i);
                } else ++after;
            });
            before = block_sum_double(before, fs->dred);
            const double more_d = block_sum_double((double)after, fs->dred);
            if (threadIdx.x == 0) ts0->d[1][tm.rank] = before, ts0->u[0][tm.rank] = more_d > 0.0 ? 1u : 0u;
            tm.sync();
            if (tm.rank == 0) {
                const unsigned int n = fs->n_list;
                if (n > FS_CAP) {                        // too many for the list: divide this bin
                    if (threadIdx.x == 0) fs->status = 2;
                } else {
                    // sort the bin's keys, largest first (bitonic over the next power of two, padded with zeros)
                    unsigned int m = 1u;
                    while (m < n) m <<= 1;
                    for (unsigned int i = n + threadIdx.x; i < m; i += blockDim.x) fs->list[i] = 0ull;
                    __syncthreads();
                    for (unsigned int k = 2; k <= m; k <<= 1) {
                        for (unsigned int j = k >> 1; j > 0; j >>= 1) {
                            for (unsigned int i = threadIdx.x; i < m; i += blockDim.x) {
                                const unsigned int l = i ^ j;
                                if (l > i) {
                                    const unsigned long long a = fs->list[i], c = fs->list[l];
                                    const bool desc = (i & k) == 0;
                                    if (desc ? (a < c) : (a > c)) { fs->list[i] = c; fs->list[l] = a; }
                                }
                            }
                            __syncthreads();
                        }
                    }
                    for (unsigned int i = threadIdx.x; i < n; i += blockDim.x) {
                        const unsigned long long key = fs->list[i];
                        fs->lp[i] = weight(value_of_key(key), (int)(0xFFFFFFFFu - (unsigned int)(key & 0xFFFFFFFFull)));
                    }
                    __syncthreads();
                    if (threadIdx.x == 0) {
                        double cum = 0.0;
                        unsigned int more = 0u;
                        for (int r = 0; r < tm.n; ++r) cum += ts->d[1][r], more += ts->u[0][r];
                        int v = -1;
                        if (strict ? (cum > target) : (cum >= target)) {
                            // the crossing lies before this bin: the nearest bin with candidates before it, if any
                            int b = bsel - 1;
                            while (b >= 0 && fs->cnt[b] == 0u) --b;
                            if (b >= 0) { fs->bin = b; v = 0; }
                            else if (lo > 0.f) v = 3;        // before a divided bin's range: not ours to settle
                        }
                        if (v < 0) {
                            unsigned int i = 0;
                            for (; i < n; ++i) {
                                cum += (double)fs->lp[i];
                                if (strict ? (cum > target) : (cum >= target)) break;
                            }
                            if (i < n) { fs->key = fs->list[i]; fs->cum = cum; v = 1; }
                            else if (more > 0u) {
                                int b = bsel + 1;
                                while (b < FS_BINS && fs->cnt[b] == 0u) ++b;
                                if (b < FS_BINS) { fs->bin = b; v = 0; }
                                else v = 3;                  // candidates after the range: not ours to settle
                            } else if (n > 0u) { fs->key = fs->list[n - 1]; fs->cum = cum; v = 1; }   // never reached: the last candidate
                            else v = 3;
                        }
                        fs->status = v;
                        fs->n_list = 0u;
                    }
                }
            }
            tm.sync();
            st = fs0->status;
            if (st != 0) break;
        }
        if (st == 0) st = 3;                             // six tries and still moving: give up
        if (st == 1) {
            *out_key = fs0->key;
            *out_cum = fs0->cum;
            tm.sync();
            return true;
        }
        if (st != 2) { tm.sync(); return false; }
        // divide the chosen bin: its range of x in FS_BINS bins (the open last bin up to the largest x of the row)
        const int bsel = fs0->bin;
        const float blo = lo + (float)bsel / inv_w;
        const float bhi = (open_end && bsel == FS_BINS - 1) ? x_max : lo + (float)(bsel + 1) / inv_w;
        tm.sync();
        if (!(bhi > blo)) return false;
        lo = blo;
        inv_w = (float)FS_BINS / (bhi - blo);
        open_end = false;
        if (!isfinite(inv_w)) return false;
    }
    return false;
}

struct SampleParams {
    float temperature;
    int top_k;          // 0: off
    float top_p;        // >= 1: off
    float min_p;        // <= 0: off
};

__global__ void __launch_bounds__(SAMPLE_THREADS, 1)
sample_rows_kernel(const float* __restrict__ logits, int ld, int vocab, SampleParams sp_launch,
                   const float* __restrict__ params_dev, const float* __restrict__ draws, int* __restrict__ out,
                   int* __restrict__ err) {
    // temperature, top_k, top_p, min_p: from device memory where given (a captured graph then serves any of them)
    SampleParams sp = sp_launch;
    if (params_dev != nullptr) {
        sp.temperature = params_dev[0];
        sp.top_k = (int)params_dev[1];
        sp.top_p = params_dev[2];
        sp.min_p = params_dev[3];
    }
    __shared__ SelectShared sh;
    __shared__ FastShared fs;
    __shared__ TeamSlots ts;
    Team tm;
    tm.n = (int)cg::this_cluster().num_blocks();
    tm.rank = (int)cg::this_cluster().block_rank();
    const int row_index = blockIdx.x / tm.n;
    {   // slices of whole groups of four columns
        const int per = (((vocab + tm.n - 1) / tm.n) + 3) & ~3;
        tm.begin = min(vocab, tm.rank * per);
        tm.end = min(vocab, tm.begin + per);
    }
    TeamSlots* ts0 = tm.at0(&ts);
    const float* row = logits + (size_t)row_index * ld;

    // maximum and minimum logit and finiteness
    float mx = -CUDART_INF_F, mn = CUDART_INF_F;
    bool bad = false;
    for_each_in_slice(row, tm, [&](float v, int) {
        if (!isfinite(v)) bad = true;
        mx = fmaxf(mx, v);
        mn = fminf(mn, v);
    });
    if (bad) atomicOr(err, SAMPLE_ERR_NONFINITE);
    {
        const float bmx = block_max(mx, fs.lp), bmn = -block_max(-mn, fs.lp);     // lp: free until a selection runs
        if (threadIdx.x == 0) ts0->f[0][tm.rank] = bmx, ts0->f[1][tm.rank] = bmn, ts0->u[1][tm.rank] = 0u;
        const int any_bad = __syncthreads_or(bad ? 1 : 0);
        if (threadIdx.x == 0 && any_bad) ts0->u[1][tm.rank] = 1u;
    }
    tm.sync();
    mx = -CUDART_INF_F, mn = CUDART_INF_F;
    unsigned int team_bad = 0u;
    for (int r = 0; r < tm.n; ++r) {
        mx = fmaxf(mx, ts0->f[0][r]);
        mn = fminf(mn, ts0->f[1][r]);
        team_bad |= ts0->u[1][r];
    }
    const float T = sp.temperature;
    const float max_scaled = mx / T;
    // the place of a value in the order, as a distance from the maximum (what the exponential is taken of)
    const float inv_T = 1.0f / T, x_zero = mx * inv_T;
    // monotone in v and never negative, which is all it has to be (the product rounded on its own: fused into the
    // subtraction, the maximum's own place would come out as the product's rounding error, of either sign)
    auto xof = [=](float v) { return fmaxf(x_zero - __fmul_rn(v, inv_T), 0.f); };
    const float x_max = xof(mn);
    if (team_bad != 0u || !isfinite(x_max)) {              // not a number, or infinite: the error is set; no choice
        if (tm.rank == 0 && threadIdx.x == 0) out[row_index] = 0;
        tm.sync();                                         // nobody leaves while block 0's slots may still be read
        return;
    }

    unsigned long long floor_key = 0ull;
    unsigned long long key;
    double cum;
    // The selection in the digits of the key, by block 0 alone over the whole row, where the fast one gives up.
    auto select_slow = [&](unsigned long long floor, double target, int strict, auto weight) {
        FastShared* fs0 = tm.at0(&fs);
        if (tm.rank == 0) {
            unsigned long long k;
            double c;
            select_by_mass(row, vocab, floor, target, strict, weight, &sh, &k, &c);
            if (threadIdx.x == 0) fs.key = k, fs.cum = c;
        }
        tm.sync();
        key = fs0->key;
        cum = fs0->cum;
        tm.sync();
    };
    // top_k: the k-th candidate in order becomes the floor
    if (sp.top_k > 0 && sp.top_k < vocab) {
        auto one = [](float, int) { return 1.0f; };
        auto one_at = [](float) { return 1.0f; };
        if (!select_fast(row, tm, 0ull, (double)sp.top_k, 0, xof, x_max, one, one_at, &fs, &ts, &key, &cum))
            select_slow(0ull, (double)sp.top_k, 0, one);
        floor_key = key;
    }
    auto raw_weight = [=](float v, int) { return expf(v / T - max_scaled); };
    // A short list of candidates (top_k of a few hundred at most, the usual case): their keys are collected and
    // sorted once, and the rest of the way (the sum, min_p, top_p, the draw) is walked along that list by one
    // thread of block 0, with the same arithmetic as the passes over the row below.
    if (floor_key != 0ull && sp.top_k > 0 && sp.top_k <= SAMPLE_LIST_WALK) {
        FastShared* fs0 = tm.at0(&fs);
        if (tm.rank == 0 && threadIdx.x == 0) fs.n_list = 0u;
        tm.sync();
        for_each_in_slice(row, tm, [&](float v, int i) {
            const unsigned long long ck = composite_key(v, i);
            if (ck >= floor_key) {
                const unsigned int slot = atomicAdd(&fs0->n_list, 1u);
                if (slot < FS_CAP) fs0->list[slot] = ck;
            }
        });
        tm.sync();
        if (tm.rank == 0) {
            const unsigned int n = min(fs.n_list, (unsigned int)FS_CAP);      // top_k keys: the k largest
            unsigned int m = 1u;
            while (m < n) m <<= 1;
            for (unsigned int i = n + threadIdx.x; i < m; i += blockDim.x) fs.list[i] = 0ull;
            __syncthreads();
            for (unsigned int k = 2; k <= m; k <<= 1) {
                for (unsigned int j = k >> 1; j > 0; j >>= 1) {
                    for (unsigned int i = threadIdx.x; i < m; i += blockDim.x) {
                        const unsigned int l = i ^ j;
                        if (l > i) {
                            const unsigned long long a = fs.list[i], c = fs.list[l];
                            const bool desc = (i & k) == 0;
                            if (desc ? (a < c) : (a > c)) { fs.list[i] = c; fs.list[l] = a; }
                        }
                    }
                    __syncthreads();
                }
            }
            for (unsigned int i = threadIdx.x; i < n; i += blockDim.x) fs.lp[i] = raw_weight(value_of_key(fs.list[i]), 0);
            __syncthreads();
            if (threadIdx.x == 0) {
                double total_d = 0.0;
                for (unsigned int i = 0; i < n; ++i) total_d += (double)fs.lp[i];
                const float total = (float)total_d;
                if (!(total > 0.f) || !isfinite(total)) {
                    atomicOr(err, SAMPLE_ERR_EMPTY);
                    out[row_index] = 0;
                } else {
                    unsigned int cand = n;                              // the candidates are list[0 .. cand)
                    float renorm = 1.0f, renorm2 = 1.0f;
                    if (sp.min_p > 0.f) {
                        const float thr = sp.min_p * (1.0f / total);
                        double sum = 0.0;
                        unsigned int kept = 0;
                        for (unsigned int i = 0; i < cand; ++i) {       // values descend, so do the probabilities
                            const float pr = fs.lp[i] / total;
                            if (pr >= thr) { sum += (double)pr; kept = i + 1; }
                        }
                        if (kept > 0 && sum > 0.0) { cand = kept; renorm = (float)sum; }
                    }
                    if (sp.top_p < 1.0f) {
                        double c = 0.0;
                        unsigned int i = 0;
                        for (; i < cand; ++i) {
                            c += (double)(fs.lp[i] / total / renorm);
                            if (c >= (double)sp.top_p) break;
                        }
                        if (i < cand) cand = i + 1;                     // never reached: all of them, with their sum
                        renorm2 = (float)c;
                    }
                    const double draw = (double)draws[row_index];
                    double c = 0.0;
                    unsigned int i = 0;
                    for (; i < cand; ++i) {
                        c += (double)(fs.lp[i] / total / renorm / renorm2);
                        if (c > draw) break;
                    }
                    if (i >= cand) i = cand - 1;                        // never reached: the last candidate
                    out[row_index] = (int)(0xFFFFFFFFu - (unsigned int)(fs.list[i] & 0xFFFFFFFFull));
                }
            }
        }
        tm.sync();
        return;
    }
    // softmax weights and their sum over the candidates
    double part = 0.0;
    for_each_in_slice(row, tm, [&](float v, int i) {
        if (composite_key(v, i) >= floor_key) part += (double)raw_weight(v, i);
    });
    part = block_sum_double(part, fs.dred);
    if (threadIdx.x == 0) ts0->d[2][tm.rank] = part;
    tm.sync();
    double total_d = 0.0;
    for (int r = 0; r < tm.n; ++r) total_d += ts0->d[2][r];
    const float total = (float)total_d;
    if (!(total > 0.f) || !isfinite(total)) {
        if (tm.rank == 0 && threadIdx.x == 0) { atomicOr(err, SAMPLE_ERR_EMPTY); out[row_index] = 0; }
        tm.sync();
        return;
    }
    float renorm = 1.0f;                 // successive renormalisations: p = w / total / renorm...
    float renorm2 = 1.0f;
    // min_p: keep p >= min_p * p_max, p_max being the first candidate's probability
    if (sp.min_p > 0.f) {
        const float pmax = 1.0f / total;             // weight of the maximum is exp(0) = 1
        const float thr = sp.min_p * pmax;
        unsigned long long kmin = ~0ull;
        double s = 0.0;
        for_each_in_slice(row, tm, [&](float v, int i) {
            const unsigned long long ck = composite_key(v, i);
            if (ck < floor_key) return;
            const float p = raw_weight(v, i) / total;
            if (p >= thr) { s += (double)p; kmin = ck < kmin ? ck : kmin; }
        });
        s = block_sum_double(s, fs.dred);
        {   // the smallest key over the block
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long ok = __shfl_xor_sync(0xffffffffu, kmin, o);
                kmin = ok < kmin ? ok : kmin;
            }
            __syncthreads();
            if (lane == 0) fs.list[warp] = kmin;          // list: free until a selection runs
            __syncthreads();
            if (threadIdx.x == 0) {
                for (int w = 1; w < nw; ++w) kmin = fs.list[w] < kmin ? fs.list[w] : kmin;
                ts0->d[3][tm.rank] = s;
                ts0->k[0][tm.rank] = kmin;
            }
        }
        tm.sync();
        double s_all = 0.0;
        unsigned long long k_all = ~0ull;
        for (int r = 0; r < tm.n; ++r) {
            s_all += ts0->d[3][r];
            k_all = ts0->k[0][r] < k_all ? ts0->k[0][r] : k_all;
        }
        if (k_all != ~0ull && s_all > 0.0) {
            floor_key = k_all;
            renorm = (float)s_all;
        }
    }
    // top_p: shortest prefix whose cumulative probability reaches top_p
    if (sp.top_p < 1.0f) {
        auto p1 = [=](float v, int) { return raw_weight(v, 0) / total / renorm; };
        const float c1 = 1.0f / total / renorm;
        auto a1 = [=](float x) { return __expf(-x) * c1; };
        if (!select_fast(row, tm, floor_key, (double)sp.top_p, 0, xof, x_max, p1, a1, &fs, &ts, &key, &cum))
            select_slow(floor_key, (double)sp.top_p, 0, p1);
        floor_key = key;
        renorm2 = (float)cum;
    }
    // the draw
    auto p2 = [=](float v, int) { return raw_weight(v, 0) / total / renorm / renorm2; };
    const float c2 = 1.0f / total / renorm / renorm2;
    auto a2 = [=](float x) { return __expf(-x) * c2; };
    const double draw = (double)draws[row_index];
    if (!select_fast(row, tm, floor_key, draw, 1, xof, x_max, p2, a2, &fs, &ts, &key, &cum))
        select_slow(floor_key, draw, 1, p2);
    if (tm.rank == 0 && threadIdx.x == 0) out[row_index] = (int)(0xFFFFFFFFu - (unsigned int)(key & 0xFFFFFFFFull));
    tm.sync();                                             // block 0's shared memory stays until every block has read it
}

// The draws of a step on the device: row r of a one-token step feeds the token at position
// positions[r], so the history its next token is drawn for has positions[r] + 1 tokens, and the
// draw is the reference's stream at that place: the top 24 bits of
// splitmix64(seed + (length + 1) * golden) / 2^24 (src/inference.rs:6160-6180). The seed is read
// from device memory, so one captured graph serves every seed.
__global__ void draws_at_kernel(const int* __restrict__ positions, const unsigned long long* __restrict__ seed,
                                float* __restrict__ draws, int rows) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const unsigned long long length = (unsigned long long)(positions[r] + 1);
    unsigned long long z = *seed + (length + 1ull) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    draws[r] = (float)(z >> 40) / (float)(1u << 24);
}

extern "C" int cml_draws_at(const int* positions, const unsigned long long* seed, float* draws, int rows, void* stream) {
    if (rows <= 0) return 0;
    draws_at_kernel<<<(rows + 127) / 128, 128, 0, (cudaStream_t)stream>>>(positions, seed, draws, rows);
    return cml_launch_status();
}

// draws[r] in [0, 1) is computed by the host from the seed and the length of the history.
// `params_dev` (may be null): four floats in device memory, temperature, top_k (0: off), top_p (1: off), min_p (0: off),
// read by the kernel instead of the arguments.
extern "C" int cml_sample_rows(const float* logits, int ld, int rows, int vocab, float temperature, int top_k,
                               float top_p, float min_p, const float* params_dev, const float* draws, int* out, int* err,
                               void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || (params_dev == nullptr && !(temperature > 0.f))) return CML_ERR_BAD_SIZE;
    SampleParams sp;
    sp.temperature = temperature;
    sp.top_k = top_k;
    sp.top_p = top_p;
    sp.min_p = min_p;
    // A row of 32k columns or more is shared by a cluster of up to 8 blocks, a shorter one by fewer; a block of
    // 1,024 threads takes a multiprocessor to itself, so no more blocks than there are multiprocessors.
    int team = vocab >= 32768 ? 8 : (vocab >= 8192 ? 4 : 1);
    while (team > 1 && rows * team > cml_sm_count()) team >>= 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(rows * team));
    cfg.blockDim = dim3(SAMPLE_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)team;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t le = cudaLaunchKernelEx(&cfg, sample_rows_kernel, logits, ld, vocab, sp, params_dev, draws, out, err);
    if (le != cudaSuccess) return (int)le;
    return cml_launch_status();
}

// ------------------------------------------------------------------------------------
// The greedy choice again, for callers that cannot allocate: the same kernel with its two
// words per row in a fixed array of this library instead of a buffer the caller brings.
// See argmax_static.h for who needs this and for the rules of use.
#include "argmax_static.h"
#include <mutex>
#include <stdio.h>

// 2 words x 8 bytes per row. File-scope device memory: zero when the module is loaded.
static __device__ __align__(256) unsigned long long g_argmax_static_words[2 * CML_ARGMAX_STATIC_MAX_ROWS];

#define CML_MAX_DEVICES 64
static unsigned long long* g_argmax_static_ptr[CML_MAX_DEVICES];     // device address per GPU, looked up once
static std::mutex g_argmax_static_mutex;

static void refuse(char* msg, int msg_len, const char* text) {
    if (msg && msg_len > 0) snprintf(msg, (size_t)msg_len, "%s", text);
}

extern "C" int cml_argmax_rows_static(const float* logits, int ld, int rows, int vocab, int* out, int* err,
                                      void* stream, char* msg, int msg_len) {
    if (msg && msg_len > 0) msg[0] = 0;
    if (rows <= 0) return 0;
    if (rows > CML_ARGMAX_STATIC_MAX_ROWS) {
        if (msg && msg_len > 0)
            snprintf(msg, (size_t)msg_len, "cml_argmax_rows_static: %d rows exceed the fixed scratch of %d rows; "
                     "split the call or use cml_argmax_rows with a buffer of your own", rows, CML_ARGMAX_STATIC_MAX_ROWS);
        return CML_ARGMAX_STATIC_TOO_MANY_ROWS;
    }
    if (!logits || !out || !err || vocab <= 0 || ld < vocab) {
        refuse(msg, msg_len, "cml_argmax_rows_static: null pointer, vocab <= 0 or ld < vocab");
        return CML_ARGMAX_STATIC_BAD_ARGUMENT;
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        refuse(msg, msg_len, "cml_argmax_rows_static: cudaGetDevice failed");
        return (int)e;
    }
    if (dev < 0 || dev >= CML_MAX_DEVICES) {
        refuse(msg, msg_len, "cml_argmax_rows_static: device index beyond the table of this library");
        return CML_ARGMAX_STATIC_BAD_ARGUMENT;
    }
    unsigned long long* words;
    {
        // Set-up, once per GPU and with that GPU current: in host code the array's name is
        // only a handle, the kernel needs the address the symbol has on this device.
        std::lock_guard<std::mutex> lock(g_argmax_static_mutex);
        if (!g_argmax_static_ptr[dev]) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_argmax_static_words);
            if (e != cudaSuccess) {
                refuse(msg, msg_len, "cml_argmax_rows_static: cudaGetSymbolAddress failed");
                return (int)e;
            }
            g_argmax_static_ptr[dev] = (unsigned long long*)p;
        }
        words = g_argmax_static_ptr[dev];
    }
    cudaStream_t s = (cudaStream_t)stream;
    // the words of these rows must start at zero, whatever an earlier call left
    e = cudaMemsetAsync(words, 0, (size_t)rows * 2 * sizeof(unsigned long long), s);
    if (e != cudaSuccess) {
        refuse(msg, msg_len, "cml_argmax_rows_static: clearing the scratch words failed");
        return (int)e;
    }
    const int blocks = argmax_blocks(rows, vocab);
    argmax_rows_kernel<<<dim3(blocks, rows), 256, 0, s>>>(logits, ld, vocab, out, err, words);
    e = cudaGetLastError();
    if (e != cudaSuccess) refuse(msg, msg_len, "cml_argmax_rows_static: the kernel launch failed");
    return (int)e;
}
