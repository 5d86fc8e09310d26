// Attention over the paged cache for any head size, head count and grouping, in float
// arithmetic on the CUDA cores: the kernel of the true 32-bit path, and the path that
// takes every shape the tensor-core kernels refuse. Prefill and decode are the same kernel
// with different tilings.
//
// It replaces attention_decode (src/cuda_resident.rs:1587), attention_batched (:1994) and
// the split-K family attn_sk_* (:2332-2487). The arithmetic follows the reference's
// per-head routine (src/inference.rs:23945-24025): score = (q . k) * scale, running
// maximum, exp(score - max), and probabilities times values; query head h reads kv head
// h / (heads / kv_heads) (src/inference/diagnostic_config.rs:300-317). A query at absolute
// position p sees keys lo..p with lo = max(0, p - window + 1) when a window is set, else 0.
//
// Work split: one block handles `rows_per_tile` consecutive new tokens of one sequence,
// `heads_per_cta` query heads of one kv head, and one contiguous range of key pages
// (`n_splits` ranges; partial results are merged by attn_combine_kernel). One warp owns one
// token and 1, 2 or 4 of its heads (a key or value read from shared memory then serves all of
// them; a decode step, with few pairs, gives every head its own warp); the block shares each
// key/value page through shared memory, two pages deep: the next page is fetched while the warps
// work on this one.
#include "attention_common.cuh"

__device__ __forceinline__ void cp_async16_f(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit_f() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait_f() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One page of keys and values into a stage of shared memory. Keys lie in rows of hd floats whose
// 16-byte chunks are exchanged by the row number (chunk c of row j at c ^ (j & mask)), so that the
// lanes of a warp, each reading its own key row, meet different banks without padding; values lie
// as they are. Float pages come by cp.async (the next page is on its way while this one is worked
// on); other types are converted on the way.
template <typename T>
__device__ __forceinline__ void attn_stage_page(float* Ks, float* Vs, const T* kp, const T* vp, size_t base, int hd, int mask) {
    const int chunks = hd >> 2;
    // (row j, chunk c) of this thread's first piece, then steps of blockDim.x pieces without a division
    const int dj = blockDim.x / chunks, dc = blockDim.x - dj * chunks;
    int j = threadIdx.x / chunks, c = threadIdx.x - j * chunks;
    for (int idx = threadIdx.x; idx < CML_PAGE * chunks; idx += blockDim.x) {
        float* kd = Ks + ((size_t)j * chunks + (c ^ (j & mask))) * 4;
        float* vd = Vs + (size_t)idx * 4;
        if (sizeof(T) == 4) {
            cp_async16_f(kd, reinterpret_cast<const float*>(kp) + base + (size_t)idx * 4);
            cp_async16_f(vd, reinterpret_cast<const float*>(vp) + base + (size_t)idx * 4);
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                kd[e] = to_f32(kp[base + (size_t)idx * 4 + e]);
                vd[e] = to_f32(vp[base + (size_t)idx * 4 + e]);
            }
        }
        j += dj;
        c += dc;
        if (c >= chunks) {
            c -= chunks;
            ++j;
        }
    }
}

template <typename T, int NACC, int R>
__global__ void attn_paged_simt_kernel(AttnParams p) {
    extern __shared__ __align__(16) float smem[];
    pdl_wait();
    pdl_launch_dependents();
    const int hd = p.head_dim;
    const int chunks = hd >> 2;
    const int mask = (chunks & 7) == 0 ? 7 : 3;
    const int n_warps = blockDim.x >> 5;
    const int stage_floats = 2 * CML_PAGE * hd;          // keys, then values
    const int n_stages = p.n_stages;                     // 2, or 1 where two pages of this head size do not fit
    float* Qs = smem + n_stages * stage_floats;          // [warps][R][hd]
    float* Ps = Qs + n_warps * R * hd;                   // [warps][PAGE][R]

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
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps_per_row = p.heads_per_cta / R;       // a warp owns R heads of one token
    const int r_local = warp / warps_per_row;
    const int hg0 = chunk * p.heads_per_cta + (warp - r_local * warps_per_row) * R;
    const bool valid = (r_local < p.rows_per_tile) && (q0 + r_local < n_new) && (hg0 < group);
    const int head0 = kvh * group + hg0;
    const int row = row0 + q0 + r_local;
    const int pos = start + q0 + r_local;
    const int rows_in_tile = min(p.rows_per_tile, n_new - q0);
    const int kend = start + q0 + rows_in_tile;                       // exclusive
    const int kbeg = p.window > 0 ? max(0, start + q0 - p.window + 1) : 0;
    const int b_first = kbeg / CML_PAGE;
    const int b_last = (kend + CML_PAGE - 1) / CML_PAGE;              // exclusive
    const int per = (b_last - b_first + p.n_splits - 1) / p.n_splits;
    const int sb = b_first + split * per;
    const int se = min(b_last, sb + per);
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;

    const T* q = (const T*)p.q;
    if (valid) {
#pragma unroll
        for (int rr = 0; rr < R; ++rr)                                // a head beyond the group: zeros, never stored
            for (int d = lane; d < hd; d += 32)
                Qs[(warp * R + rr) * hd + d] = hg0 + rr < group ? to_f32(q[(size_t)row * p.q_stride + (head0 + rr) * hd + d]) : 0.f;
    }

    float m[R], l[R];
    float acc[R][NACC];
#pragma unroll
    for (int rr = 0; rr < R; ++rr) {
        m[rr] = -CUDART_INF_F;
        l[rr] = 0.f;
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[rr][i] = 0.f;
    }

    const T* kp = (const T*)p.k_pages;
    const T* vp = (const T*)p.v_pages;
    auto page_base = [&](int b) {
        const int page = p.block_table[(size_t)seq * p.max_blocks + b];
        return ((size_t)page * p.n_kv_heads + kvh) * CML_PAGE * hd;
    };
    if (n_stages == 2 && sb < se) attn_stage_page<T>(smem, smem + CML_PAGE * hd, kp, vp, page_base(sb), hd, mask);
    cp_async_commit_f();
    for (int b = sb; b < se; ++b) {
        float* Ks = smem + (n_stages == 2 ? ((b - sb) & 1) * stage_floats : 0);
        float* Vs = Ks + CML_PAGE * hd;
        if (n_stages == 2) {
            if (b + 1 < se) {          // the other stage was read in the round before; all warps are past it
                float* Kn = smem + ((b + 1 - sb) & 1) * stage_floats;
                attn_stage_page<T>(Kn, Kn + CML_PAGE * hd, kp, vp, page_base(b + 1), hd, mask);
            }
            cp_async_commit_f();
            cp_async_wait_f<1>();
        } else {
            attn_stage_page<T>(Ks, Vs, kp, vp, page_base(b), hd, mask);
            cp_async_commit_f();
            cp_async_wait_f<0>();
        }
        __syncthreads();
        const int live_rows = kend - b * CML_PAGE;                  // rows past the end may hold anything:
        if (live_rows < CML_PAGE) {                                 // their values must not meet a zero probability
            for (int idx = threadIdx.x + live_rows * hd; idx < CML_PAGE * hd; idx += blockDim.x) Vs[idx] = 0.f;
            __syncthreads();
        }
        if (valid) {
            // A lane takes two keys of the page; a key's chunk, once read, serves the R heads of the warp.
            const int k0 = b * CML_PAGE + lane, k1 = k0 + 32;
            const float4* q4 = reinterpret_cast<const float4*>(Qs + (size_t)warp * R * hd);
            const float4* ka = reinterpret_cast<const float4*>(Ks) + (size_t)lane * chunks;
            const float4* kb = reinterpret_cast<const float4*>(Ks) + (size_t)(lane + 32) * chunks;
            const int x0 = lane & mask, x1 = (lane + 32) & mask;
            float s0[R], s1[R];
#pragma unroll
            for (int rr = 0; rr < R; ++rr) s0[rr] = 0.f, s1[rr] = 0.f;
#pragma unroll 4
            for (int c = 0; c < chunks; ++c) {                      // chunks is a multiple of 4: whole rounds
                const float4 a = ka[c ^ x0], bb = kb[c ^ x1];
#pragma unroll
                for (int rr = 0; rr < R; ++rr) {
                    const float4 qq = q4[rr * chunks + c];
                    s0[rr] = fmaf(qq.x, a.x, s0[rr]); s0[rr] = fmaf(qq.y, a.y, s0[rr]); s0[rr] = fmaf(qq.z, a.z, s0[rr]); s0[rr] = fmaf(qq.w, a.w, s0[rr]);
                    s1[rr] = fmaf(qq.x, bb.x, s1[rr]); s1[rr] = fmaf(qq.y, bb.y, s1[rr]); s1[rr] = fmaf(qq.z, bb.z, s1[rr]); s1[rr] = fmaf(qq.w, bb.w, s1[rr]);
                }
            }
            const bool in0 = (k0 >= lo) && (k0 <= pos), in1 = (k1 >= lo) && (k1 <= pos);
            if (__any_sync(0xffffffffu, in0 || in1)) {                  // a visible key in this page (the same for every head)
                float* pw = Ps + (size_t)warp * CML_PAGE * R;
#pragma unroll
                for (int rr = 0; rr < R; ++rr) {
                    const float t0 = in0 ? s0[rr] * p.scale : -CUDART_INF_F;
                    const float t1 = in1 ? s1[rr] * p.scale : -CUDART_INF_F;
                    const float bm = warp_max(fmaxf(t0, t1));
                    const float mn = fmaxf(m[rr], bm);
                    const float corr = (m[rr] == -CUDART_INF_F) ? 0.f : expf(m[rr] - mn);
                    const float p0 = in0 ? expf(t0 - mn) : 0.f;
                    const float p1 = in1 ? expf(t1 - mn) : 0.f;
                    l[rr] = l[rr] * corr + warp_sum(p0 + p1);
#pragma unroll
                    for (int i = 0; i < NACC; ++i) acc[rr][i] *= corr;
                    pw[lane * R + rr] = p0;
                    pw[(lane + 32) * R + rr] = p1;
                    m[rr] = mn;
                }
                __syncwarp();
                const int jend = min(CML_PAGE, live_rows);
#pragma unroll 4
                for (int j = 0; j < jend; ++j) {
                    float pj[R];
                    if (R == 4) {
                        const float4 t = *reinterpret_cast<const float4*>(pw + j * 4);
                        pj[0] = t.x; pj[1 % R] = t.y; pj[2 % R] = t.z; pj[3 % R] = t.w;
                    } else if (R == 2) {
                        const float2 t = *reinterpret_cast<const float2*>(pw + j * 2);
                        pj[0] = t.x; pj[1 % R] = t.y;
                    } else {
                        pj[0] = pw[j];
                    }
                    const float* vr = Vs + j * hd;
#pragma unroll
                    for (int i = 0; i < NACC; ++i) {
                        const int d = lane + 32 * i;
                        if (d < hd) {
                            const float v = vr[d];
#pragma unroll
                            for (int rr = 0; rr < R; ++rr) acc[rr][i] = fmaf(pj[rr], v, acc[rr][i]);
                        }
                    }
                }
                __syncwarp();
            }
        }
        __syncthreads();               // this stage is free for the page after the next
    }
    cp_async_wait_f<0>();
    if (!valid) return;
#pragma unroll
    for (int rr = 0; rr < R; ++rr) {
        if (hg0 + rr >= group) break;
        const int head = head0 + rr;
        if (p.n_splits == 1) {
            T* o = (T*)p.out + (size_t)row * p.out_stride + head * hd;
            const float inv = 1.0f / l[rr];
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                const int d = lane + 32 * i;
                if (d < hd) o[d] = from_f32<T>(acc[rr][i] * inv);
            }
        } else {
            float* o = p.partial + (((size_t)row * p.n_heads + head) * p.n_splits + split) * (hd + 2);
            if (lane == 0) {
                o[0] = m[rr];
                o[1] = l[rr];
            }
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                const int d = lane + 32 * i;
                if (d < hd) o[2 + d] = acc[rr][i];
            }
        }
    }
}

// Decode (one new token per tile): a block owns the token, H (2 or 4) query heads of one kv head and a range
// of key pages, like the kernel above, but its four warps share a page by keys, not by heads: warp w takes
// keys 16 w .. 16 w + 15 of every page for all H heads, a lane one key and H / 2 heads. A key chunk read from
// shared memory then serves H heads and a value row H heads, a third of the shared-memory traffic of one
// warp per head, which is what bounds this kernel when the cache streams from HBM. Every warp keeps its own
// running maximum, sum and output rows per head; at the end the four are merged in warp order through shared
// memory and written as the kernel above writes them.
template <typename T, int NACC, int H>
__global__ void __launch_bounds__(128) attn_decode_simt_kernel(AttnParams p) {
    constexpr int HL = H / 2;                            // heads of a lane
    extern __shared__ __align__(16) float smem[];
    pdl_launch_dependents();
    const int hd = p.head_dim;
    const int chunks = hd >> 2;
    const int mask = (chunks & 7) == 0 ? 7 : 3;
    const int qld = hd + 4;                              // rows of Qs a bank group apart
    const int stage_floats = 2 * CML_PAGE * hd;          // keys, then values
    const int n_stages = p.n_stages;
    float* Qs = smem + n_stages * stage_floats;          // [H][hd + 4]
    float* Ps = Qs + H * qld;                            // [4 warps][16 keys][H]
    float* Ms = Ps + 4 * 16 * H;                         // [4 warps][H][2 + hd]: maximum, sum, output row

    const int tile = blockIdx.x;
    const int seq = p.tile_seq[tile];
    const int q0 = p.tile_q0[tile];
    const int kvh = blockIdx.y / p.head_chunks;
    const int chunk = blockIdx.y - kvh * p.head_chunks;
    const int split = blockIdx.z;
    const int start = p.seq_start[seq];
    const int row = p.seq_row0[seq] + q0;
    const int group = p.n_heads / p.n_kv_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hg0 = chunk * H;
    const int head0 = kvh * group + hg0;
    const int pos = start + q0;
    const int kend = pos + 1;
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int b_first = lo / CML_PAGE;
    const int b_last = (kend + CML_PAGE - 1) / CML_PAGE;
    const int per = (b_last - b_first + p.n_splits - 1) / p.n_splits;
    const int sb = b_first + split * per;
    const int se = min(b_last, sb + per);

    float m[H], l_own[HL];                               // l_own: the sums of this lane's keys for its own heads
    float acc[H][NACC];
#pragma unroll
    for (int hl = 0; hl < HL; ++hl) l_own[hl] = 0.f;
#pragma unroll
    for (int h = 0; h < H; ++h) {
        m[h] = -CUDART_INF_F;
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[h][i] = 0.f;
    }
    const T* kp = (const T*)p.k_pages;
    const T* vp = (const T*)p.v_pages;
    auto page_base = [&](int b) {
        const int page = p.block_table[(size_t)seq * p.max_blocks + b];
        return ((size_t)page * p.n_kv_heads + kvh) * CML_PAGE * hd;
    };
    const bool low = lane < 16;
    const int kk = 16 * warp + (lane & 15);              // this lane's key within a page
    const int x = kk & mask;
    // Pages below the token's own were written by earlier steps: the first one (two, with two stages) is asked
    // for before the wait on the kernel that writes this step's key and value; the block table, positions and
    // lengths are the step's inputs, in place before its first kernel started.
    constexpr int MAX_STAGES = 2;
    bool early[MAX_STAGES] = {false, false};
    if (n_stages > 1) {
#pragma unroll
        for (int u = 0; u < MAX_STAGES; ++u) {
            early[u] = u < n_stages && sb + u < se && (sb + u + 1) * CML_PAGE <= pos;
            if (early[u]) attn_stage_page<T>(smem + u * stage_floats, smem + u * stage_floats + CML_PAGE * hd, kp, vp, page_base(sb + u), hd, mask);
        }
    }
    pdl_wait();
    {
        const T* q = (const T*)p.q;
        for (int i = threadIdx.x; i < H * hd; i += blockDim.x) {
            const int h = i / hd, d = i - h * hd;           // a head beyond the group: zeros, never stored
            Qs[h * qld + d] = hg0 + h < group ? to_f32(q[(size_t)row * p.q_stride + (head0 + h) * hd + d]) : 0.f;
        }
    }
    if (n_stages > 1) {
#pragma unroll
        for (int u = 0; u < MAX_STAGES; ++u) {
            if (u >= n_stages) break;
            if (!early[u] && sb + u < se)
                attn_stage_page<T>(smem + u * stage_floats, smem + u * stage_floats + CML_PAGE * hd, kp, vp, page_base(sb + u), hd, mask);
            cp_async_commit_f();                          // one group per page, empty ones included
        }
    }
    int stage = 0;                                        // of page b
    for (int b = sb; b < se; ++b) {
        float* Ks = smem + stage * stage_floats;
        float* Vs = Ks + CML_PAGE * hd;
        if (n_stages == 2) {
            cp_async_wait_f<1>();                         // all but the newest group: page b is here
        } else {
            attn_stage_page<T>(Ks, Vs, kp, vp, page_base(b), hd, mask);
            cp_async_commit_f();
            cp_async_wait_f<0>();
        }
        __syncthreads();
        const int key = b * CML_PAGE + kk;
        const bool in = key >= lo && key <= pos;
        if (__any_sync(0xffffffffu, in)) {
            const float4* ka = reinterpret_cast<const float4*>(Ks) + (size_t)kk * chunks;
            const float* qh = Qs + (low ? 0 : HL) * qld;
            // four chunks a round (the head size is a multiple of 16), even and odd chunks in sums of their own:
            // the loads of a round are in flight together and the chains of dependent FMAs half as long
            float sc[HL], sd[HL];
#pragma unroll
            for (int hl = 0; hl < HL; ++hl) sc[hl] = 0.f, sd[hl] = 0.f;
            for (int c0 = 0; c0 < chunks; c0 += 4) {
                float4 a[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) a[u] = ka[(c0 + u) ^ x];
#pragma unroll
                for (int hl = 0; hl < HL; ++hl) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const float4 qq = *reinterpret_cast<const float4*>(qh + hl * qld + 4 * (c0 + u));
                        float& acc_s = (u & 1) ? sd[hl] : sc[hl];
                        acc_s = fmaf(qq.x, a[u].x, acc_s); acc_s = fmaf(qq.y, a[u].y, acc_s);
                        acc_s = fmaf(qq.z, a[u].z, acc_s); acc_s = fmaf(qq.w, a[u].w, acc_s);
                    }
                }
            }
#pragma unroll
            for (int hl = 0; hl < HL; ++hl) sc[hl] += sd[hl];
            // The reference m[h] the exponentials are taken against follows the maximum lazily: it moves only
            // when a score of the warp stands more than 5.5 above it (probabilities up to e^5.5 are harmless in
            // float), which one vote finds out; the reductions over lanes, the rescaling of the sums and output rows
            // then happen on the first page and rarely after. Numerator and denominator share the reference, so
            // the result is the same. A lane sums the probabilities of its own keys; the lanes meet at the end.
            float t[HL];
            bool move = false;
#pragma unroll
            for (int hl = 0; hl < HL; ++hl) {
                t[hl] = in ? sc[hl] * p.scale : -CUDART_INF_F;
                const float mo = low ? m[hl] : m[HL + hl];
                move = move || (in && (mo == -CUDART_INF_F || t[hl] > mo + 5.5f));
            }
            if (__any_sync(0xffffffffu, move)) {
#pragma unroll
                for (int hl = 0; hl < HL; ++hl) {
                    float bm = t[hl];                                // maximum over the 16 keys of this half warp
#pragma unroll
                    for (int o = 8; o >= 1; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o));
                    const float other = __shfl_xor_sync(0xffffffffu, bm, 16);
                    const float bm_lo = low ? bm : other, bm_hi = low ? other : bm;  // heads hl and HL + hl
                    const float mn_lo = fmaxf(m[hl], bm_lo), mn_hi = fmaxf(m[HL + hl], bm_hi);
                    const float c_lo = (m[hl] == -CUDART_INF_F) ? 0.f : expf(m[hl] - mn_lo);
                    const float c_hi = (m[HL + hl] == -CUDART_INF_F) ? 0.f : expf(m[HL + hl] - mn_hi);
                    m[hl] = mn_lo;
                    m[HL + hl] = mn_hi;
                    l_own[hl] *= low ? c_lo : c_hi;
#pragma unroll
                    for (int i = 0; i < NACC; ++i) {
                        acc[hl][i] *= c_lo;
                        acc[HL + hl][i] *= c_hi;
                    }
                }
            }
            float* pw = Ps + warp * 16 * H;
#pragma unroll
            for (int hl = 0; hl < HL; ++hl) {
                const float pr = in ? expf(t[hl] - (low ? m[hl] : m[HL + hl])) : 0.f;
                pw[(lane & 15) * H + (low ? 0 : HL) + hl] = pr;
                l_own[hl] += pr;
            }
            __syncwarp();
            // value rows past the end may hold anything: they are read (every load is unconditional, so that all
            // of them can be in flight together) and replaced by zero
            const int jend = kend - (b * CML_PAGE + 16 * warp);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                float pj[H];
                if (H == 4) {
                    const float4 v4 = *reinterpret_cast<const float4*>(pw + j * 4);
                    pj[0] = v4.x; pj[1] = v4.y; pj[2 % H] = v4.z; pj[3 % H] = v4.w;
                } else {
                    const float2 v2 = *reinterpret_cast<const float2*>(pw + j * 2);
                    pj[0] = v2.x; pj[1] = v2.y;
                }
                const float* vr = Vs + (16 * warp + j) * hd;
#pragma unroll
                for (int i = 0; i < NACC; ++i) {
                    const int d = min(lane + 32 * i, hd - 1);        // a clamped lane's sums are never stored
                    const float vv = vr[d];
                    const float v = j < jend ? vv : 0.f;
#pragma unroll
                    for (int h = 0; h < H; ++h) acc[h][i] = fmaf(pj[h], v, acc[h][i]);
                }
            }
            __syncwarp();
        }
        __syncthreads();               // this stage is free for the page after the next
        if (n_stages > 1) {
            if (b + n_stages < se) attn_stage_page<T>(Ks, Vs, kp, vp, page_base(b + n_stages), hd, mask);
            cp_async_commit_f();
            stage = stage + 1 == n_stages ? 0 : stage + 1;
        }
    }
    cp_async_wait_f<0>();
    // the lanes' sums over the 16 keys of a half warp, then every lane has those of all heads
    float l[H];
#pragma unroll
    for (int hl = 0; hl < HL; ++hl) {
        float sum = l_own[hl];
#pragma unroll
        for (int o = 8; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float other = __shfl_xor_sync(0xffffffffu, sum, 16);
        l[hl] = low ? sum : other;
        l[HL + hl] = low ? other : sum;
    }
    // the four warps' ranges of keys into one, in warp order
#pragma unroll
    for (int h = 0; h < H; ++h) {
        float* mine = Ms + (size_t)(warp * H + h) * (2 + hd);
        if (lane == 0) {
            mine[0] = m[h];
            mine[1] = l[h];
        }
#pragma unroll
        for (int i = 0; i < NACC; ++i) {
            const int d = lane + 32 * i;
            if (d < hd) mine[2 + d] = acc[h][i];
        }
    }
    __syncthreads();
    for (int h = warp; h < H; h += 4) {
        if (hg0 + h >= group) break;
        float M = -CUDART_INF_F;
        for (int w = 0; w < 4; ++w) M = fmaxf(M, Ms[(size_t)(w * H + h) * (2 + hd)]);
        float L = 0.f, wgt[4];
        for (int w = 0; w < 4; ++w) {
            const float mw = Ms[(size_t)(w * H + h) * (2 + hd)];
            wgt[w] = (mw == -CUDART_INF_F) ? 0.f : expf(mw - M);
            L += wgt[w] * Ms[(size_t)(w * H + h) * (2 + hd) + 1];
        }
        const int head = head0 + h;
        float* po = p.partial + (((size_t)row * p.n_heads + head) * p.n_splits + split) * (hd + 2);
        T* o = (T*)p.out + (size_t)row * p.out_stride + head * hd;
        if (p.n_splits > 1 && lane == 0) {
            po[0] = M;
            po[1] = L;
        }
        for (int d = lane; d < hd; d += 32) {
            float a = 0.f;
            for (int w = 0; w < 4; ++w) a += wgt[w] * Ms[(size_t)(w * H + h) * (2 + hd) + 2 + d];
            if (p.n_splits > 1) po[2 + d] = a;
            else o[d] = from_f32<T>(a / L);
        }
    }
}

// Pages a block of the decode kernel keeps in shared memory: two, or one where two do not fit. (Three, with two
// blocks an SM instead of three, were slower at batch 8: 1.65 against 1.60 ms a float decode step.)
static int cml_attn_decode_stages(size_t stage, size_t rest) { return 2 * stage + rest <= 200 * 1024 ? 2 : 1; }

template <typename T>
static int launch_attn(const AttnParams& p_in, int heads_per_warp, int n_tiles, int n_rows, cudaStream_t s) {
    const int hd = p_in.head_dim;
    const int R = heads_per_warp;
    if (R == 0) {
        // a decode step's tiling: four warps share every page by keys, all of them on the block's 2 or 4 heads
        const int H = p_in.heads_per_cta;
        if (p_in.rows_per_tile != 1 || (H != 2 && H != 4)) return CML_ERR_BAD_SIZE;
        if (p_in.n_splits > 1 && p_in.partial == nullptr) return CML_ERR_BAD_SIZE;
        const size_t rest = ((size_t)H * (hd + 4) + 64 * H + (size_t)4 * H * (2 + hd)) * sizeof(float);
        const size_t stage = (size_t)2 * CML_PAGE * hd * sizeof(float);
        AttnParams p = p_in;
        p.n_stages = cml_attn_decode_stages(stage, rest);
        const size_t smem = p.n_stages * stage + rest;
        if (smem > 227 * 1024) return CML_ERR_BAD_SIZE;
        const int nacc = (hd + 31) / 32;
        dim3 grid(n_tiles, p.n_kv_heads * p.head_chunks, p.n_splits);
        cudaError_t e = cudaSuccess;
#define CML_ATTD(N, HH)                                                                                    \
    do {                                                                                                   \
        e = cml_allow_smem<attn_decode_simt_kernel<T, N, HH>>(smem);                                       \
        if (e != cudaSuccess) return (int)e;                                                               \
        launch_pdl(attn_decode_simt_kernel<T, N, HH>, grid, dim3(128), smem, s, p);                        \
    } while (0)
#define CML_ATTD_N(HH)                                                                                     \
    do {                                                                                                   \
        if (nacc <= 1) CML_ATTD(1, HH);                                                                    \
        else if (nacc <= 2) CML_ATTD(2, HH);                                                               \
        else if (nacc <= 4) CML_ATTD(4, HH);                                                               \
        else if (nacc <= 8) CML_ATTD(8, HH);                                                               \
        else return CML_ERR_BAD_SIZE;                                                                      \
    } while (0)
        if (H == 4) CML_ATTD_N(4);
        else CML_ATTD_N(2);
#undef CML_ATTD_N
#undef CML_ATTD
        e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
        if (p.n_splits > 1) {
            launch_pdl(attn_combine_kernel<T>, dim3(n_rows * p.n_heads), dim3(hd >= 128 ? 128 : 64), 0, s,
                       (const float*)p.partial, (T*)p.out, p.out_stride, p.n_heads, hd, p.n_splits);
            e = cudaGetLastError();
        }
        return (int)e;
    }
    if ((R != 1 && R != 2 && R != 4) || p_in.heads_per_cta % R != 0) return CML_ERR_BAD_SIZE;
    const int warps = p_in.rows_per_tile * (p_in.heads_per_cta / R);
    if (warps < 1 || warps > 32) return CML_ERR_BAD_SIZE;
    const size_t rest = ((size_t)warps * R * hd + (size_t)warps * R * CML_PAGE) * sizeof(float);
    const size_t stage = (size_t)2 * CML_PAGE * hd * sizeof(float);
    AttnParams p = p_in;
    p.n_stages = 2 * stage + rest <= 200 * 1024 ? 2 : 1;
    const size_t smem = p.n_stages * stage + rest;
    if (smem > 227 * 1024) return CML_ERR_BAD_SIZE;
    const int nacc = (hd + 31) / 32;
    dim3 grid(n_tiles, p.n_kv_heads * p.head_chunks, p.n_splits);
    dim3 block(warps * 32);
    cudaError_t e = cudaSuccess;
#define CML_ATTN(N, RR)                                                                                    \
    do {                                                                                                   \
        e = cml_allow_smem<attn_paged_simt_kernel<T, N, RR>>(smem);                                        \
        if (e != cudaSuccess) return (int)e;                                                               \
        launch_pdl(attn_paged_simt_kernel<T, N, RR>, grid, block, smem, s, p);                             \
    } while (0)
#define CML_ATTN_N(RR)                                                                                     \
    do {                                                                                                   \
        if (nacc <= 1) CML_ATTN(1, RR);                                                                    \
        else if (nacc <= 2) CML_ATTN(2, RR);                                                               \
        else if (nacc <= 4) CML_ATTN(4, RR);                                                               \
        else if (nacc <= 8) CML_ATTN(8, RR);                                                               \
        else return CML_ERR_BAD_SIZE;                                                                      \
    } while (0)
    if (R == 4) CML_ATTN_N(4);
    else if (R == 2) CML_ATTN_N(2);
    else CML_ATTN_N(1);
#undef CML_ATTN_N
#undef CML_ATTN
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (p.n_splits > 1) {
        launch_pdl(attn_combine_kernel<T>, dim3(n_rows * p.n_heads), dim3(hd >= 128 ? 128 : 64), 0, s,
                   (const float*)p.partial, (T*)p.out, p.out_stride, p.n_heads, hd, p.n_splits);
        e = cudaGetLastError();
    }
    return (int)e;
}

// `partial` must hold n_rows * n_heads * n_splits * (head_dim + 2) floats when n_splits > 1.
// A block has rows_per_tile * heads_per_cta / heads_per_warp warps (at most 32); heads_per_warp is 1, 2 or 4
// and divides heads_per_cta. heads_per_warp 0 (tiles of one row, 2 or 4 heads a block): the decode kernel whose
// warps share a page by keys.
extern "C" long cml_attn_simt_smem_bytes(int head_dim, int rows_per_tile, int heads_per_cta, int heads_per_warp) {
    const size_t stage = (size_t)2 * CML_PAGE * head_dim * sizeof(float);
    size_t rest;
    if (heads_per_warp == 0)
        rest = ((size_t)heads_per_cta * (head_dim + 4) + 64 * heads_per_cta + (size_t)4 * heads_per_cta * (2 + head_dim)) * sizeof(float);
    else
        rest = (size_t)rows_per_tile * heads_per_cta * (head_dim + CML_PAGE) * sizeof(float);
    if (heads_per_warp == 0) return (long)(cml_attn_decode_stages(stage, rest) * stage + rest);
    return (long)((2 * stage + rest <= 200 * 1024 ? 2 : 1) * stage + rest);
}
extern "C" int cml_attn_paged_simt(const void* q, int q_stride, void* out, int out_stride, int dtype,
                                   const void* k_pages, const void* v_pages, const int* block_table, int max_blocks,
                                   const int* tile_seq, const int* tile_q0, int n_tiles, const int* seq_row0,
                                   const int* seq_start, const int* seq_new, int n_rows, int n_heads, int n_kv_heads,
                                   int head_dim, int rows_per_tile, int heads_per_cta, int heads_per_warp, int head_chunks,
                                   int n_splits, int window, float scale, float* partial, void* stream) {
    if (n_tiles <= 0 || n_rows <= 0) return 0;
    if (head_dim <= 0 || head_dim > 256 || (head_dim & 15) || n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return CML_ERR_BAD_SIZE;
    if (((uintptr_t)k_pages | (uintptr_t)v_pages) & 15) return CML_ERR_BAD_ALIGN;
    if (n_splits < 1 || (n_splits > 1 && partial == nullptr)) return CML_ERR_BAD_SIZE;
    if (heads_per_cta * head_chunks < n_heads / n_kv_heads) return CML_ERR_BAD_SIZE;
    AttnParams p;
    p.q = q; p.q_stride = q_stride; p.out = out; p.out_stride = out_stride;
    p.k_pages = k_pages; p.v_pages = v_pages; p.block_table = block_table; p.max_blocks = max_blocks;
    p.tile_seq = tile_seq; p.tile_q0 = tile_q0; p.seq_row0 = seq_row0; p.seq_start = seq_start; p.seq_new = seq_new;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim;
    p.rows_per_tile = rows_per_tile; p.heads_per_cta = heads_per_cta; p.head_chunks = head_chunks;
    p.n_splits = n_splits; p.window = window; p.scale = scale; p.partial = partial; p.tickets = nullptr; p.n_stages = 2;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CML_DTYPE_F32) return launch_attn<float>(p, heads_per_warp, n_tiles, n_rows, s);
    if (dtype == CML_DTYPE_BF16) return launch_attn<bf16>(p, heads_per_warp, n_tiles, n_rows, s);
    return CML_ERR_BAD_DTYPE;
}
