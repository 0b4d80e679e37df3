// Softmax attention over the paged KV cache with the options the Llama path does not have: biases on q/k/v, an RMS norm
// over the whole q (and k) projection, rotation of the first `rot_dims` dimensions of a head in adjacent pairs,
// a tanh cap on the scores, a block-local causal mask (a query sees the keys of its own block of `chunk` positions),
// a zero-score sink in the softmax denominator, a sigmoid gate per head on the output, any head sizes (the value size
// may differ from the query/key size); and, each optional: a sliding window, a penalty per head and unit of distance,
// a learned sink score per head, key and value rows wider than the heads (so that both can share one page array).
// The row kernel serves prompt portions and single decoded tokens alike: a warp owns one (row, head) and walks the keys
// it sees 32 at a time; scores, softmax and accumulation are fp32. For bf16 pages there are two tensor-core forms of
// the same arithmetic further down: 64 consecutive rows of a prompt portion per CTA, and (decoded tokens) the query
// heads of one key/value group as the rows of a tile, with the keys cut into slices.
// Cache element type XT = bf16 or fp32. Pages hold `bs` tokens: K [blocks, G, bs, k_row], V [blocks, G, bs, v_row].
#include "common.cuh"

#include "../../include/atx_b200.h"

namespace atx {

template <typename XT>
__device__ __forceinline__ float ldx(const XT* p, long long i);
template <>
__device__ __forceinline__ float ldx<float>(const float* p, long long i) {
    return p[i];
}
template <>
__device__ __forceinline__ float ldx<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
    return __bfloat162float(p[i]);
}
__device__ __forceinline__ void stx(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void stx(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }
// Two adjacent elements in one access; i is even and p + i is aligned to the pair.
__device__ __forceinline__ void stx2(float* p, long long i, float a, float b) {
    *reinterpret_cast<float2*>(p + i) = make_float2(a, b);
}
__device__ __forceinline__ void stx2(__nv_bfloat16* p, long long i, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p + i) = __floats2bfloat162_rn(a, b);
}

// ---- bias, whole-projection RMS norm, partial rotation, page scatter ----------------------------------------------
// One block per row. rot: [max_pos, rot_dims] fp32, cos of the rot_dims/2 angles then their sines.
template <typename XT>
__global__ void __launch_bounds__(256)
qk_prepare_kernel(const float* __restrict__ proj, long long ld, int q_off, int k_off, int v_off,
                  const XT* __restrict__ bq, const XT* __restrict__ bk, const XT* __restrict__ bv,
                  const XT* __restrict__ wq, const XT* __restrict__ wk, const float* __restrict__ rot, int rot_dims,
                  const int* __restrict__ positions, const int* __restrict__ slots, XT* __restrict__ q_out,
                  XT* __restrict__ k_cache, XT* __restrict__ v_cache, int H, int G, int D, int Vd, int bs, float eps) {
    extern __shared__ float sm[];
    __shared__ float red[2][32];
    pdl_launch_dependents();
    pdl_wait();
    const long long t = blockIdx.x;
    const int slot = slots[t];
    if (slot < 0) return;  // padded row
    const int nq = H * D, nk = G * D;
    float* sq = sm;
    float* sk = sm + nq;
    const float* row = proj + t * ld;
    float ssq = 0.f, ssk = 0.f;
    // pairs in one access when the row, both offsets and the outputs keep a pair aligned (the usual case)
    const bool pairs = ((q_off | k_off | nq | D) & 1) == 0 && (ld & 1) == 0 &&
                       (reinterpret_cast<unsigned long long>(proj) & 7) == 0 &&
                       (reinterpret_cast<unsigned long long>(q_out) & 7) == 0 &&
                       (reinterpret_cast<unsigned long long>(k_cache) & 7) == 0;
    if (pairs) {
        #pragma unroll 4
        for (int i = 2 * threadIdx.x; i < nq; i += 2 * blockDim.x) {
            float2 v = *reinterpret_cast<const float2*>(row + q_off + i);
            if (bq) {
                v.x += ldx(bq, i);
                v.y += ldx(bq, i + 1);
            }
            *reinterpret_cast<float2*>(sq + i) = v;
            ssq += v.x * v.x + v.y * v.y;
        }
        #pragma unroll 4
        for (int i = 2 * threadIdx.x; i < nk; i += 2 * blockDim.x) {
            float2 v = *reinterpret_cast<const float2*>(row + k_off + i);
            if (bk) {
                v.x += ldx(bk, i);
                v.y += ldx(bk, i + 1);
            }
            *reinterpret_cast<float2*>(sk + i) = v;
            ssk += v.x * v.x + v.y * v.y;
        }
    } else {
        for (int i = threadIdx.x; i < nq; i += blockDim.x) {
            float v = row[q_off + i];
            if (bq) v += ldx(bq, i);
            sq[i] = v;
            ssq += v * v;
        }
        for (int i = threadIdx.x; i < nk; i += blockDim.x) {
            float v = row[k_off + i];
            if (bk) v += ldx(bk, i);
            sk[i] = v;
            ssk += v * v;
        }
    }
    ssq = warp_sum(ssq);
    ssk = warp_sum(ssk);
    if ((threadIdx.x & 31) == 0) {
        red[0][threadIdx.x >> 5] = ssq;
        red[1][threadIdx.x >> 5] = ssk;
    }
    __syncthreads();
    float tq = 0.f, tk = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) {
        tq += red[0][i];
        tk += red[1][i];
    }
    const float rq = wq ? rsqrtf(tq / static_cast<float>(nq) + eps) : 1.f;
    const float rk = wk ? rsqrtf(tk / static_cast<float>(nk) + eps) : 1.f;
    const int pos = positions[t];
    const float* cs = rot + static_cast<long long>(pos) * rot_dims;
    const int half = rot_dims / 2;
    const int blk = slot / bs, off = slot - blk * bs;
    // q and k: work items are pairs of adjacent dimensions
    #pragma unroll 4
    for (int e = threadIdx.x; e < (nq + nk) / 2; e += blockDim.x) {
        const bool isq = e < nq / 2;
        const int p = isq ? e : e - nq / 2;  // pair index inside q or k
        const int i0 = 2 * p;
        const int head = i0 / D, d = i0 - head * D;
        float a, b;
        if (isq) {
            a = sq[i0] * rq;
            b = sq[i0 + 1] * rq;
            if (wq) {
                a *= ldx(wq, i0);
                b *= ldx(wq, i0 + 1);
            }
        } else {
            a = sk[i0] * rk;
            b = sk[i0 + 1] * rk;
            if (wk) {
                a *= ldx(wk, i0);
                b *= ldx(wk, i0 + 1);
            }
        }
        if (d < rot_dims) {
            const float c = cs[d / 2], s = cs[half + d / 2];
            const float ra = a * c - b * s, rb = b * c + a * s;
            a = ra;
            b = rb;
        }
        if (isq) {
            if (pairs) {
                stx2(q_out, t * nq + i0, a, b);
            } else {
                stx(q_out, t * nq + i0, a);
                stx(q_out, t * nq + i0 + 1, b);
            }
        } else {
            const long long base = ((static_cast<long long>(blk) * G + head) * bs + off) * D + d;
            if (pairs) {
                stx2(k_cache, base, a, b);
            } else {
                stx(k_cache, base, a);
                stx(k_cache, base + 1, b);
            }
        }
    }
    for (int i = threadIdx.x; i < G * Vd; i += blockDim.x) {
        const int head = i / Vd, d = i - head * Vd;
        float v = row[v_off + i];
        if (bv) v += ldx(bv, i);
        stx(v_cache, ((static_cast<long long>(blk) * G + head) * bs + off) * Vd + d, v);
    }
}

// ---- attention ---------------------------------------------------------------------------------------------------
constexpr int kMaxVdPerLane = 16;  // Vd <= 512; the kernel is instantiated for 2, 4, 8 and 16 value elements per lane

template <typename XT, int NV>
__global__ void __launch_bounds__(128)
attn_local_kernel(const XT* __restrict__ q, const XT* __restrict__ k_cache, const XT* __restrict__ v_cache,
                  const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ tok_seq,
                  const int* __restrict__ positions, const float* __restrict__ gate, long long ldg,
                  XT* __restrict__ out, long long ldo, int H, int G, int D, int Vd, int bs, float scale, float softcap,
                  int chunk, int sink, float out_scale, long long k_row, long long v_row, int window,
                  const float* __restrict__ slopes, const float* __restrict__ sinks, int keep_first, int sigmoid_w,
                  const float* __restrict__ bias, int gate_elem) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long t = blockIdx.x;
    const int h = blockIdx.y * 4 + warp;
    const int s = tok_seq[t];
    if (s < 0 || h >= H) return;
    const int g = h / (H / G);
    const int pos = positions[t];
    int lo = chunk > 0 ? (pos / chunk) * chunk : 0;
    if (window > 0) lo = max(lo, pos - window + 1);   // sliding window: the row itself and the window - 1 tokens before it
    const float slope = slopes ? slopes[h] : 0.f;
    const float hb = bias ? bias[h] : 0.f;   // added to every score of the head
    float* sq = sm + warp * D;
    for (int d = lane; d < D; d += 32) sq[d] = ldx(q, (t * H + h) * D + d) * scale;
    __syncwarp();
    const int* bt = block_tables + static_cast<long long>(s) * max_blocks;
    // the sink is a key with a fixed score (0, or a learned number per head) and no value: the running maximum starts
    // at that score and the denominator at 1
    const bool has_sink = sink || sinks;
    float m = has_sink ? (sinks ? sinks[h] : 0.f) : -INFINITY, l = has_sink ? 1.f : 0.f;
    float acc[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[i] = 0.f;
    // keys come in two ranges: the first positions that stay visible below the window's edge, then the window itself
    const int kept_end = min(keep_first, lo);
    for (int range = kept_end > 0 ? 0 : 1; range < 2; ++range) {
    const int k_begin = range == 0 ? 0 : lo, k_last = range == 0 ? kept_end - 1 : pos;
    for (int k0 = k_begin; k0 <= k_last; k0 += 32) {
        const int kp = k0 + lane;
        float sc = -INFINITY;
        long long vbase = 0;
        if (kp <= k_last) {
            const int blk = bt[kp / bs];
            const long long tokslot = (static_cast<long long>(blk) * G + g) * bs + (kp % bs);
            const XT* kr = k_cache + tokslot * k_row;
            vbase = tokslot * v_row;
            float dot = 0.f;
            for (int d = 0; d < D; ++d) dot = fmaf(sq[d], ldx(kr, d), dot);
            sc = softcap > 0.f ? softcap * tanhf(dot / softcap) : dot;
            sc -= slope * static_cast<float>(pos - kp);   // penalty per unit of distance
            sc += hb;
        }
        float p;
        if (sigmoid_w) {   // every visible key weighs sigmoid(score) by itself: no maximum, no sum
            p = (kp <= k_last) ? 1.f / (1.f + expf(-sc)) : 0.f;
        } else {
            const float mt = fmaxf(m, warp_max(sc));
            const float corr = (m == -INFINITY) ? 0.f : expf(m - mt);
            p = (kp <= k_last) ? expf(sc - mt) : 0.f;
            l = l * corr + warp_sum(p);
#pragma unroll
            for (int i = 0; i < NV; ++i) acc[i] *= corr;
            m = mt;
        }
        const int nk = min(32, k_last - k0 + 1);
        for (int j = 0; j < nk; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long long vb = __shfl_sync(0xffffffffu, vbase, j);
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int d = lane + 32 * i;
                if (d < Vd) acc[i] = fmaf(pj, ldx(v_cache, vb + d), acc[i]);
            }
        }
    }
    }
    float gmul = sigmoid_w ? out_scale : out_scale / l;
    if (gate && !gate_elem) gmul *= 1.f / (1.f + expf(-gate[t * ldg + h]));
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int d = lane + 32 * i;
        if (d >= Vd) continue;
        float v = acc[i] * gmul;
        if (gate && gate_elem) v *= 1.f / (1.f + expf(-gate[t * ldg + static_cast<long long>(h) * Vd + d]));
        stx(out, t * ldo + static_cast<long long>(h) * Vd + d, v);
    }
}

// ---- prompt portions on the tensor cores (bf16) -----------------------------------------------------------------------
// One CTA = 64 consecutive rows of one sequence's portion x one query head; a warp owns 16 rows. Key tiles of 64
// positions are gathered from the pages into shared memory; S = Q K^T and O += P V run on mma.sync m16n8k16 (bf16 in,
// fp32 accumulate), everything between (scale, tanh cap, block-local causal mask, running maximum and sum with the
// zero-score sink, rescale of O) is fp32 in registers. Key/value tiles arrive by cp.async into two stages, the next
// tile in flight while the current one is multiplied; the query tile is staged in the second stage's space before the
// pipeline starts (its fragments then live in registers), which keeps a CTA at four tiles of shared memory and three
// CTAs on an SM. The portion's sequences are listed as (first row, rows, first position); a CTA finds its tile by
// walking that list.
__device__ __forceinline__ void cp_async16_zfill(void* smem_dst, const void* gsrc, bool valid) {
    const uint32_t sz = valid ? 16u : 0u;   // source size 0: sixteen bytes of zeros, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(sz) : "memory");
}
__device__ __forceinline__ float tanh_via_exp(float x) {
    const float t = __expf(2.f * x);          // inf for large x: 2 / inf = 0 -> 1; 0 for very negative x -> -1
    return 1.f - __fdividef(2.f, t + 1.f);
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

constexpr int kTcRows = 64, kTcKeys = 64;

// D and VD are the tile's key and value widths; the heads' own sizes d_real <= D and vd_real <= VD (multiples of 8) are
// run-time values: the columns between are zero in shared memory, so one instance serves every size up to its own.
// A token's key row has k_row elements and its value row v_row (keys and values may share one page array). window > 0
// cuts the keys below p - window + 1; slopes[h] (p - j) is taken off the score; sinks[h] is the learned score of the sink.
//
// DEC: the decode form of the same kernel. A CTA takes ONE token, one key/value head and one slice of the keys; the tile's
// rows are the query heads that share that key/value head (at most 64), all at the token's position, each with its own
// slope and sink, so K and V are read once for the whole group. Slices (gridDim.z) write unnormalised partial outputs
// with their running maximum and sum to `ws` and attn_split_merge_kernel folds them; the sink counts in slice 0 only.
// Rows are listed by tok_seq / positions (one entry per token) instead of (first row, rows, first position) triples.
//
// SIG: every visible key weighs sigmoid(score + bias[h]) by itself (no running maximum, no sum, no division at the end;
// slices of the decode form simply add up). keep_first: keys at positions below it stay visible under the window's lower
// edge; they are walked as tiles of their own in front of the window's tiles, up to where the window's tiles begin.
// gate_elem: the gate holds a number per output element ([., H * vd_real]) instead of one per head.
template <int D, int VD, bool DEC, bool SIG>
__global__ void __launch_bounds__(128, (D <= 64 ? 4 : (D <= 128 ? 3 : 2)))
attn_local_tc_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                     const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_tables, int max_blocks,
                     const int* __restrict__ seq_start, const int* __restrict__ seq_count,
                     const int* __restrict__ seq_pos0, int n_seqs, const float* __restrict__ gate, long long ldg,
                     __nv_bfloat16* __restrict__ out, long long ldo, int H, int G, int bs, float scale, float softcap,
                     int chunk, int sink, float out_scale, int d_real, int vd_real, long long k_row, long long v_row,
                     int window, const float* __restrict__ slopes, const float* __restrict__ sinks,
                     const int* __restrict__ tok_seq, const int* __restrict__ positions, float* __restrict__ ws,
                     int keep_first, const float* __restrict__ bias, int gate_elem) {
    constexpr int LQ = D + 8, LV = VD + 8;     // padded rows: ldmatrix without bank conflicts, 16-byte aligned
    extern __shared__ __align__(16) unsigned char smem_raw[];
    static_assert(kTcRows == kTcKeys, "the query tile is staged in a key stage");
    __nv_bfloat16* sKs = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [2][kTcKeys][LQ]
    __nv_bfloat16* sVs = sKs + 2 * kTcKeys * LQ;                        // [2][kTcKeys][LV]
    __nv_bfloat16* sQ = sKs + kTcKeys * LQ;                             // = key stage 1, until the pipeline starts
    pdl_launch_dependents();
    pdl_wait();
    int tile = gridDim.x - 1 - blockIdx.x, s = 0;   // later tiles see more keys: the heaviest start first
    const int group = H / G;
    int h, g, nrows, p0, p1;
    long long row0;
    if constexpr (DEC) {
        row0 = blockIdx.x;                 // the token
        s = tok_seq[row0];
        if (s < 0) return;                 // padded row
        g = blockIdx.y;
        h = g * group;                     // first head of the group; row r of the tile is head h + r
        nrows = group;
        p0 = p1 = positions[row0];
    } else {
        for (; s < n_seqs; ++s) {
            const int nt = (seq_count[s] + kTcRows - 1) / kTcRows;
            if (tile < nt) break;
            tile -= nt;
        }
        if (s >= n_seqs) return;
        h = blockIdx.y;
        g = h / group;
        row0 = seq_start[s] + tile * kTcRows;
        nrows = min(kTcRows, seq_count[s] - tile * kTcRows);
        p0 = seq_pos0[s] + tile * kTcRows;
        p1 = p0 + nrows - 1;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto lower_edge = [&](int p) -> int {   // first key a query at p sees
        int e = chunk > 0 ? (p / chunk) * chunk : 0;
        if (window > 0) e = max(e, p - window + 1);
        return e;
    };
    const int lo = lower_edge(p0);
    const int* bt = block_tables + static_cast<long long>(s) * max_blocks;
    const int dq8 = d_real / 8, dv8 = vd_real / 8;

    for (int c = threadIdx.x; c < kTcRows * (D / 8); c += 128) {
        const int r = c / (D / 8), part = c - r * (D / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nrows && part < dq8) {
            const long long qrow = DEC ? row0 * H + h + r : (row0 + r) * H + h;
            v = __ldg(reinterpret_cast<const uint4*>(q + qrow * d_real + part * 8));
        }
        *reinterpret_cast<uint4*>(sQ + r * LQ + part * 8) = v;
    }
    __syncthreads();
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
        ldsm_x4(smem_u32(sQ + (warp * 16 + (lane & 15)) * LQ + ks * 16 + (lane >> 4) * 8), qf[ks][0], qf[ks][1],
                qf[ks][2], qf[ks][3]);
    float o[VD / 8][4];
#pragma unroll
    for (int i = 0; i < VD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    constexpr float kLog2e = 1.4426950408889634f;
    const bool has_sink = sink || sinks;
    float m[2], l[2];
    // the sink: a key without a value whose score is 0 or a learned number per head (kept in the base-2 domain like the rest)
    float slope2[2], bias2[2];
    int pr[2], plo[2];
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int r = warp * 16 + (lane >> 2) + 8 * rr;
        const int hr = DEC ? h + min(r, group - 1) : h;          // the row's head
        const bool sink_here = has_sink && (!DEC || blockIdx.z == 0);   // the sink counts once: in the first slice
        m[rr] = sink_here ? (sinks ? sinks[hr] * kLog2e : 0.f) : -INFINITY;
        l[rr] = sink_here ? 1.f : 0.f;
        slope2[rr] = slopes ? slopes[hr] * kLog2e : 0.f;
        bias2[rr] = bias ? bias[hr] * kLog2e : 0.f;
        pr[rr] = DEC ? p0 : p0 + r;
        plo[rr] = lower_edge(pr[rr]);
    }
    // Scores live in the base-2 domain (s * log2 e), so that every exponential is one ex2. With a cap c:
    // c tanh(x / c) = c - 2c / (1 + exp(2x / c)), one ex2 and one rcp; the constants carry scale and log2 e.
    const float c_in = softcap > 0.f ? 2.f * scale / softcap * kLog2e : scale * kLog2e;
    const float cap2 = softcap * kLog2e;
    const int plo_last = DEC ? lo : lower_edge(p0 + warp * 16 + 15);   // lower edge of this warp's last row
    const int last_row_pos = DEC ? p0 : p0 + warp * 16 + 15, first_row_pos = DEC ? p0 : p0 + warp * 16;
    const bool warp_has_rows = warp * 16 < nrows;

    __syncthreads();   // every warp holds its query fragments: key stage 1 may be filled
    const int bs_shift = (bs & (bs - 1)) == 0 ? __ffs(bs) - 1 : -1;   // pages of 2^n tokens: shift and mask, no division
    auto slot_of = [&](int kq) -> long long {
        const int blk = bs_shift >= 0 ? kq >> bs_shift : kq / bs;
        return (static_cast<long long>(bt[blk]) * G + g) * bs + (kq - blk * bs);
    };
    // keys of a tile are valid up to kmax: the last row's position, or the end of the kept first keys
    auto load_tile = [&](int k0, int stage, int kmax) {
        __nv_bfloat16* dk = sKs + stage * kTcKeys * LQ;
        __nv_bfloat16* dv = sVs + stage * kTcKeys * LV;
        // rows past the portion and columns past the head's own size become zeros (0 x garbage would not be 0)
        for (int c = threadIdx.x; c < kTcKeys * (D / 8); c += 128) {
            const int r = c / (D / 8), part = c - r * (D / 8);
            const int kp = k0 + r;
            const bool ok = kp <= kmax && part < dq8;
            cp_async16_zfill(dk + r * LQ + part * 8, k_cache + slot_of(min(kp, kmax)) * k_row + (ok ? part * 8 : 0), ok);
        }
        for (int c = threadIdx.x; c < kTcKeys * (VD / 8); c += 128) {
            const int r = c / (VD / 8), part = c - r * (VD / 8);
            const int kp = k0 + r;
            const bool ok = kp <= kmax && part < dv8;
            cp_async16_zfill(dv + r * LV + part * 8, v_cache + slot_of(min(kp, kmax)) * v_row + (ok ? part * 8 : 0), ok);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int kept_end = min(keep_first, lo);                       // kept keys below every row's window
    const int n_kept = (kept_end + kTcKeys - 1) / kTcKeys;
    int n_tiles = n_kept + (p1 - lo) / kTcKeys + 1, it_first = 0;
    auto tile_k0 = [&](int it) { return it < n_kept ? it * kTcKeys : lo + (it - n_kept) * kTcKeys; };
    auto tile_kmax = [&](int it) { return it < n_kept ? kept_end - 1 : p1; };
    if constexpr (DEC) {   // this slice's share of the tiles
        const int per = (n_tiles + static_cast<int>(gridDim.z) - 1) / static_cast<int>(gridDim.z);
        it_first = min(n_tiles, static_cast<int>(blockIdx.z) * per);
        n_tiles = min(n_tiles, it_first + per);
    }
    if (it_first < n_tiles) load_tile(tile_k0(it_first), it_first & 1, tile_kmax(it_first));
    for (int it = it_first; it < n_tiles; ++it) {
        const int k0 = tile_k0(it);
        const bool kept_tile = it < n_kept;
        if (it + 1 < n_tiles) {
            load_tile(tile_k0(it + 1), (it + 1) & 1, tile_kmax(it + 1));
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const __nv_bfloat16* sK = sKs + (it & 1) * kTcKeys * LQ;
        const __nv_bfloat16* sV = sVs + (it & 1) * kTcKeys * LV;
        if (k0 <= last_row_pos && warp_has_rows) {   // else every key of the tile lies after this warp's rows, or the warp has none (warp-uniform)
        float sc[kTcKeys / 8][4];
#pragma unroll
        for (int i = 0; i < kTcKeys / 8; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
            for (int nb2 = 0; nb2 < kTcKeys / 16; ++nb2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(smem_u32(sK + (nb2 * 16 + (lane >> 4) * 8 + (lane & 7)) * LQ + ks * 16 + ((lane >> 3) & 1) * 8), b0,
                        b1, b2, b3);
                mma_bf16(sc[2 * nb2], qf[ks], b0, b1);
                mma_bf16(sc[2 * nb2 + 1], qf[ks], b2, b3);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
        // only tiles that reach past the warp's first row or start before its last row's block need the mask
        const bool edge = kept_tile || k0 + kTcKeys - 1 > first_row_pos || k0 < plo_last;
        if (softcap > 0.f) {
#pragma unroll
            for (int nb = 0; nb < kTcKeys / 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    sc[nb][e] = fmaf(-2.f * cap2, rcp_approx(1.f + ex2_approx(sc[nb][e] * c_in)), cap2);
            }
        } else {
#pragma unroll
            for (int nb = 0; nb < kTcKeys / 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[nb][e] *= c_in;
            }
        }
        if (slopes) {   // penalty per unit of distance between query and key
#pragma unroll
            for (int nb = 0; nb < kTcKeys / 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int col = k0 + nb * 8 + (lane & 3) * 2 + (e & 1);
                    sc[nb][e] = fmaf(-slope2[e >> 1], static_cast<float>(pr[e >> 1] - col), sc[nb][e]);
                }
            }
        }
        if (bias) {
#pragma unroll
            for (int nb = 0; nb < kTcKeys / 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[nb][e] += bias2[e >> 1];
            }
        }
        if (edge) {
            const int kend = kept_tile ? kept_end : 0x7fffffff;   // a kept tile ends where the kept keys (or the window's tiles) end
#pragma unroll
            for (int nb = 0; nb < kTcKeys / 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int col = k0 + nb * 8 + (lane & 3) * 2 + (e & 1);
                    if (col > pr[e >> 1] || col >= kend || (col < plo[e >> 1] && col >= keep_first)) sc[nb][e] = -INFINITY;
                }
            }
        }
        if constexpr (SIG) {
            // sigmoid(x) = 1 / (1 + 2^(-x log2 e)); a masked score (-inf) gives 2^inf = inf and 1 / inf = 0
#pragma unroll
            for (int nb = 0; nb < kTcKeys / 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[nb][e] = rcp_approx(1.f + ex2_approx(-sc[nb][e]));
            }
        } else {
#pragma unroll
        for (int nb = 0; nb < kTcKeys / 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], sc[nb][e]);
        }
        float corr[2], rs[2] = {0.f, 0.f};
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
            const float mn = fmaxf(m[rr], mx[rr]);
            corr[rr] = (m[rr] == -INFINITY) ? 0.f : ex2_approx(m[rr] - mn);
            m[rr] = mn;
        }
        // a row that has seen no key yet (no sink, everything masked so far): exponent base 0, so that -inf - m is -inf, not NaN
        const float mu[2] = {m[0] == -INFINITY ? 0.f : m[0], m[1] == -INFINITY ? 0.f : m[1]};
#pragma unroll
        for (int nb = 0; nb < kTcKeys / 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int rr = e >> 1;
                const float p = ex2_approx(sc[nb][e] - mu[rr]);
                sc[nb][e] = p;
                rs[rr] += p;
            }
        }
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            rs[rr] += __shfl_xor_sync(0xffffffffu, rs[rr], 1);
            rs[rr] += __shfl_xor_sync(0xffffffffu, rs[rr], 2);
            l[rr] = l[rr] * corr[rr] + rs[rr];
        }
#pragma unroll
        for (int i = 0; i < VD / 8; ++i) {
            o[i][0] *= corr[0];
            o[i][1] *= corr[0];
            o[i][2] *= corr[1];
            o[i][3] *= corr[1];
        }
        }   // softmax
#pragma unroll
        for (int kk = 0; kk < kTcKeys / 16; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
            a[1] = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
            a[2] = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
            a[3] = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
            for (int nb2 = 0; nb2 < VD / 16; ++nb2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t(smem_u32(sV + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LV + nb2 * 16 + (lane >> 4) * 8), b0,
                          b1, b2, b3);
                mma_bf16(o[2 * nb2], a, b0, b1);
                mma_bf16(o[2 * nb2 + 1], a, b2, b3);
            }
        }
        }
        __syncthreads();   // the stage is free for the tile after the next
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int r = warp * 16 + (lane >> 2) + 8 * rr;
        if (r >= nrows) continue;
        if constexpr (DEC) {
            if (gridDim.z > 1) {   // partial result of this slice: [VD outputs | maximum | sum] per (token, head, slice)
                float* w = ws + ((row0 * H + h + r) * gridDim.z + blockIdx.z) * (VD + 2);
#pragma unroll
                for (int nb = 0; nb < VD / 8; ++nb)
                    *reinterpret_cast<float2*>(w + nb * 8 + (lane & 3) * 2) = make_float2(o[nb][2 * rr], o[nb][2 * rr + 1]);
                if ((lane & 3) == 0) *reinterpret_cast<float2*>(w + VD) = make_float2(m[rr], l[rr]);
                continue;
            }
        }
        const long long orow_i = DEC ? row0 : row0 + r;
        const int oh = DEC ? h + r : h;
        float mul = SIG ? out_scale : out_scale / l[rr];
        if (gate && !gate_elem) mul *= 1.f / (1.f + __expf(-gate[orow_i * ldg + oh]));
        __nv_bfloat16* orow = out + orow_i * ldo + static_cast<long long>(oh) * vd_real + (lane & 3) * 2;
        const float* grow = (gate && gate_elem) ? gate + orow_i * ldg + static_cast<long long>(oh) * vd_real + (lane & 3) * 2 : nullptr;
#pragma unroll
        for (int nb = 0; nb < VD / 8; ++nb) {
            if (nb >= dv8) continue;
            float a = o[nb][2 * rr] * mul, b = o[nb][2 * rr + 1] * mul;
            if (gate && gate_elem) {
                a *= 1.f / (1.f + __expf(-grow[nb * 8]));
                b *= 1.f / (1.f + __expf(-grow[nb * 8 + 1]));
            }
            *reinterpret_cast<uint32_t*>(orow + nb * 8) = pack_bf16(a, b);
        }
    }
}

// key width of the smallest instance that holds D (0: none)
static int tc_key_width(int D) { return D <= 64 ? 64 : (D <= 128 ? 128 : (D <= 192 ? 192 : (D <= 256 ? 256 : 0))); }
static int tc_value_width(int Vd) { return Vd <= 64 ? 64 : (Vd <= 128 ? 128 : 0); }

// Folds the slices of the decode form: out = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), M = max_s m_s (base-2 domain).
// sigmoid_w: the slices hold plain sums of weighted values and are added as they are.
__global__ void __launch_bounds__(128)
attn_split_merge_kernel(const float* __restrict__ ws, int splits, int vd_pad, int vd_real, const int* __restrict__ tok_seq,
                        const float* __restrict__ gate, long long ldg, __nv_bfloat16* __restrict__ out, long long ldo, int H,
                        float out_scale, int sigmoid_w, int gate_elem) {
    __shared__ float wgt[64];   // weight of every slice: 2^(m_s - M) / sum (at most 64 slices)
    pdl_launch_dependents();
    pdl_wait();
    const long long t = blockIdx.x;
    const int h = blockIdx.y;
    if (tok_seq[t] < 0) return;
    const float* w = ws + (t * H + h) * splits * (vd_pad + 2);
    if (threadIdx.x < 32) {   // one warp: every lane fetches the maximum and sum of up to two slices at once
        const int lane = threadIdx.x;
        float mul = out_scale, e0 = 1.f, e1 = 1.f;
        if (!sigmoid_w) {
            float m0 = -INFINITY, l0 = 0.f, m1 = -INFINITY, l1 = 0.f;
            if (lane < splits) m0 = w[lane * (vd_pad + 2) + vd_pad], l0 = w[lane * (vd_pad + 2) + vd_pad + 1];
            if (lane + 32 < splits) m1 = w[(lane + 32) * (vd_pad + 2) + vd_pad], l1 = w[(lane + 32) * (vd_pad + 2) + vd_pad + 1];
            const float M = warp_max(fmaxf(m0, m1));
            e0 = m0 == -INFINITY ? 0.f : ex2_approx(m0 - M), e1 = m1 == -INFINITY ? 0.f : ex2_approx(m1 - M);
            const float den = warp_sum(l0 * e0 + l1 * e1);
            mul = out_scale / den;
        }
        if (gate && !gate_elem) mul *= 1.f / (1.f + __expf(-gate[t * ldg + h]));
        wgt[lane] = e0 * mul;
        wgt[lane + 32] = e1 * mul;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < vd_real; d += blockDim.x) {
        float acc = 0.f;
#pragma unroll 4
        for (int s = 0; s < splits; ++s) acc = fmaf(w[s * (vd_pad + 2) + d], wgt[s], acc);
        if (gate && gate_elem) acc *= 1.f / (1.f + __expf(-gate[t * ldg + static_cast<long long>(h) * vd_real + d]));
        out[t * ldo + static_cast<long long>(h) * vd_real + d] = __float2bfloat16_rn(acc);
    }
}

struct AttnTcArgs {
    const void *q, *k_cache, *v_cache;
    const int *block_tables, *seq_start, *seq_count, *seq_pos0;
    const float *gate, *slopes, *sinks, *bias;
    void* out;
    long long ldg, ldo, k_row, v_row;
    int max_blocks, n_seqs, max_tiles, H, G, D, Vd, bs, chunk, window, keep_first, sink, sigmoid_w, gate_elem, flags;
    float scale, softcap, out_scale;
    // decode form: rows listed by tok_seq / positions, slices of the keys, scratch for their partial results
    const int *tok_seq, *positions;
    float* ws;
    int splits;
};

template <int D, int VD, bool DEC, bool SIG>
static int launch_attn_tc(const AttnTcArgs& a, cudaStream_t stream) {
    const int smem = 2 * kTcKeys * (D + 8) * 2 + 2 * kTcKeys * (VD + 8) * 2;
    static bool attr_done = false;
    if (!attr_done && smem > 48 * 1024) {
        ATX_CUDA(cudaFuncSetAttribute(attn_local_tc_kernel<D, VD, DEC, SIG>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr_done = true;
    }
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = DEC ? dim3(a.n_seqs, a.G, a.splits) : dim3(a.max_tiles, a.H);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    if (a.flags & ATX_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    using B = __nv_bfloat16;
    ATX_CUDA(cudaLaunchKernelEx(&cfg, attn_local_tc_kernel<D, VD, DEC, SIG>, reinterpret_cast<const B*>(a.q),
                                reinterpret_cast<const B*>(a.k_cache), reinterpret_cast<const B*>(a.v_cache),
                                a.block_tables, a.max_blocks, a.seq_start, a.seq_count, a.seq_pos0, a.n_seqs, a.gate, a.ldg,
                                reinterpret_cast<B*>(a.out), a.ldo, a.H, a.G, a.bs, a.scale, a.softcap, a.chunk, a.sink,
                                a.out_scale, a.D, a.Vd, a.k_row, a.v_row, a.window, a.slopes, a.sinks, a.tok_seq, a.positions,
                                a.ws, a.keep_first, a.bias, a.gate_elem));
    if (DEC && a.splits > 1) {
        cfg.gridDim = dim3(a.n_seqs, a.H);
        cfg.dynamicSmemBytes = 0;
        ATX_CUDA(cudaLaunchKernelEx(&cfg, attn_split_merge_kernel, const_cast<const float*>(a.ws), a.splits, VD, a.Vd,
                                    a.tok_seq, a.gate, a.ldg, reinterpret_cast<B*>(a.out), a.ldo, a.H, a.out_scale,
                                    a.sigmoid_w, a.gate_elem));
    }
    return ATX_OK;
}

template <bool DEC, bool SIG>
static int dispatch_attn_tc_w(const AttnTcArgs& a, cudaStream_t st) {
    const int kw = tc_key_width(a.D), vw = tc_value_width(a.Vd);
    if (vw == 64) {
        if (kw == 64) return launch_attn_tc<64, 64, DEC, SIG>(a, st);
        if (kw == 128) return launch_attn_tc<128, 64, DEC, SIG>(a, st);
        if (kw == 192) return launch_attn_tc<192, 64, DEC, SIG>(a, st);
        return launch_attn_tc<256, 64, DEC, SIG>(a, st);
    }
    if (kw == 64) return launch_attn_tc<64, 128, DEC, SIG>(a, st);
    if (kw == 128) return launch_attn_tc<128, 128, DEC, SIG>(a, st);
    if (kw == 192) return launch_attn_tc<192, 128, DEC, SIG>(a, st);
    return launch_attn_tc<256, 128, DEC, SIG>(a, st);
}

template <bool DEC>
static int dispatch_attn_tc(const AttnTcArgs& a, cudaStream_t st) {
    return a.sigmoid_w ? dispatch_attn_tc_w<DEC, true>(a, st) : dispatch_attn_tc_w<DEC, false>(a, st);
}

static bool opts_ok(const atx_attn_opts* o) {
    return o && o->chunk >= 0 && o->window >= 0 && o->keep_first >= 0 &&
           (o->weight == ATX_ATTN_SOFTMAX || o->weight == ATX_ATTN_SIGMOID) &&
           !(o->weight == ATX_ATTN_SIGMOID && (o->sink || o->sinks));
}

}  // namespace atx

using namespace atx;

extern "C" {

int atx_qk_prepare(const float* proj, long long ld, int q_off, int k_off, int v_off, const void* bq, const void* bk,
                   const void* bv, const void* wq, const void* wk, const float* rot, int rot_dims, const int* positions,
                   const int* slots, void* q_out, void* k_cache, void* v_cache, int T, int H, int G, int D, int Vd,
                   int block_size, float eps, int dtype, int flags, atx_stream_t stream) {
    ATX_REQUIRE(proj && positions && slots && q_out && k_cache && v_cache, "atx_qk_prepare: null pointer");
    ATX_REQUIRE(T > 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && D % 2 == 0 && Vd > 0 && block_size > 0,
                "atx_qk_prepare: bad shape T=%d H=%d G=%d D=%d Vd=%d", T, H, G, D, Vd);
    ATX_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= D && (rot_dims == 0 || rot),
                "atx_qk_prepare: rot_dims=%d must be even, at most D=%d, with a table", rot_dims, D);
    const size_t smem = sizeof(float) * static_cast<size_t>(H + G) * D;
    ATX_REQUIRE(smem <= 160 * 1024, "atx_qk_prepare: (H + G) * D = %d too large", (H + G) * D);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(T);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    if (flags & ATX_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    if (dtype == ATX_DT_F32) {
        if (smem > 48 * 1024)
            ATX_CUDA(cudaFuncSetAttribute(qk_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(smem)));
        ATX_CUDA(cudaLaunchKernelEx(&cfg, qk_prepare_kernel<float>, proj, ld, q_off, k_off, v_off,
                                    reinterpret_cast<const float*>(bq), reinterpret_cast<const float*>(bk),
                                    reinterpret_cast<const float*>(bv), reinterpret_cast<const float*>(wq),
                                    reinterpret_cast<const float*>(wk), rot, rot_dims, positions, slots,
                                    reinterpret_cast<float*>(q_out), reinterpret_cast<float*>(k_cache),
                                    reinterpret_cast<float*>(v_cache), H, G, D, Vd, block_size, eps));
    } else {
        using B = __nv_bfloat16;
        if (smem > 48 * 1024)
            ATX_CUDA(cudaFuncSetAttribute(qk_prepare_kernel<B>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(smem)));
        ATX_CUDA(cudaLaunchKernelEx(&cfg, qk_prepare_kernel<B>, proj, ld, q_off, k_off, v_off,
                                    reinterpret_cast<const B*>(bq), reinterpret_cast<const B*>(bk),
                                    reinterpret_cast<const B*>(bv), reinterpret_cast<const B*>(wq),
                                    reinterpret_cast<const B*>(wk), rot, rot_dims, positions, slots,
                                    reinterpret_cast<B*>(q_out), reinterpret_cast<B*>(k_cache),
                                    reinterpret_cast<B*>(v_cache), H, G, D, Vd, block_size, eps));
    }
    return ATX_OK;
}

static atx_attn_opts softmax_opts(float scale, float softcap, int chunk, int window, const float* slopes, const float* sinks,
                                  int sink, float out_scale) {
    atx_attn_opts o = {};
    o.scale = scale, o.softcap = softcap, o.out_scale = out_scale;
    o.chunk = chunk, o.window = window, o.sink = sink, o.weight = ATX_ATTN_SOFTMAX;
    o.slopes = slopes, o.sinks = sinks;
    return o;
}

int atx_attn_local(const void* q, const void* k_cache, const void* v_cache, const int* block_tables, int max_blocks,
                   const int* tok_seq, const int* positions, const float* gate, long long ldg, void* out, long long ldo,
                   int T, int H, int G, int D, int Vd, int block_size, float scale, float softcap, int chunk, int sink,
                   float out_scale, int dtype, int flags, atx_stream_t stream) {
    return atx_attn_window(q, k_cache, v_cache, D, Vd, block_tables, max_blocks, tok_seq, positions, gate, ldg, out, ldo, T,
                           H, G, D, Vd, block_size, scale, softcap, chunk, 0, nullptr, nullptr, sink, out_scale, dtype,
                           flags, stream);
}

int atx_attn_window(const void* q, const void* k_cache, const void* v_cache, long long k_row, long long v_row,
                    const int* block_tables, int max_blocks, const int* tok_seq, const int* positions, const float* gate,
                    long long ldg, void* out, long long ldo, int T, int H, int G, int D, int Vd, int block_size,
                    float scale, float softcap, int chunk, int window, const float* slopes, const float* sinks, int sink,
                    float out_scale, int dtype, int flags, atx_stream_t stream) {
    const atx_attn_opts o = softmax_opts(scale, softcap, chunk, window, slopes, sinks, sink, out_scale);
    return atx_attn_paged(q, k_cache, v_cache, k_row, v_row, block_tables, max_blocks, tok_seq, positions, gate, ldg, out,
                          ldo, T, H, G, D, Vd, block_size, &o, dtype, flags, stream);
}

int atx_attn_paged(const void* q, const void* k_cache, const void* v_cache, long long k_row, long long v_row,
                   const int* block_tables, int max_blocks, const int* tok_seq, const int* positions, const float* gate,
                   long long ldg, void* out, long long ldo, int T, int H, int G, int D, int Vd, int block_size,
                   const atx_attn_opts* o, int dtype, int flags, atx_stream_t stream) {
    ATX_REQUIRE(q && k_cache && v_cache && block_tables && tok_seq && positions && out, "atx_attn_paged: null pointer");
    ATX_REQUIRE(opts_ok(o), "atx_attn_paged: bad options (negative sizes, unknown weight kind, or a sink with sigmoid weights)");
    ATX_REQUIRE(T > 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && Vd > 0 && Vd <= 32 * kMaxVdPerLane && block_size > 0 &&
                    k_row >= D && v_row >= Vd,
                "atx_attn_paged: bad shape T=%d H=%d G=%d D=%d Vd=%d (Vd <= %d) k_row=%lld v_row=%lld", T, H, G, D, Vd,
                32 * kMaxVdPerLane, k_row, v_row);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(T, (H + 3) / 4);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = sizeof(float) * 4 * static_cast<size_t>(D);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    if (flags & ATX_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    const int sig = o->weight == ATX_ATTN_SIGMOID ? 1 : 0;
#define ATX_ATTN_ROW_LAUNCH(XT_, NV_)                                                                                  \
    ATX_CUDA(cudaLaunchKernelEx(&cfg, attn_local_kernel<XT_, NV_>, reinterpret_cast<const XT_*>(q),                    \
                                reinterpret_cast<const XT_*>(k_cache), reinterpret_cast<const XT_*>(v_cache),          \
                                block_tables, max_blocks, tok_seq, positions, gate, ldg, reinterpret_cast<XT_*>(out),  \
                                ldo, H, G, D, Vd, block_size, o->scale, o->softcap, o->chunk, o->sink, o->out_scale,   \
                                k_row, v_row, o->window, o->slopes, o->sinks, o->keep_first, sig, o->bias,             \
                                o->gate_elem))
#define ATX_ATTN_ROW_BY_VD(XT_)                        \
    do {                                               \
        if (Vd <= 64) ATX_ATTN_ROW_LAUNCH(XT_, 2);     \
        else if (Vd <= 128) ATX_ATTN_ROW_LAUNCH(XT_, 4); \
        else if (Vd <= 256) ATX_ATTN_ROW_LAUNCH(XT_, 8); \
        else ATX_ATTN_ROW_LAUNCH(XT_, 16);             \
    } while (0)
    if (dtype == ATX_DT_F32) {
        ATX_ATTN_ROW_BY_VD(float);
    } else {
        ATX_ATTN_ROW_BY_VD(__nv_bfloat16);
    }
#undef ATX_ATTN_ROW_BY_VD
#undef ATX_ATTN_ROW_LAUNCH
    return ATX_OK;
}

int atx_attn_local_prefill_supported(int D, int Vd, int dtype) {
    return dtype == ATX_DT_BF16 && ((D == 64 && Vd == 64) || (D == 128 && Vd == 128)) ? 1 : 0;
}

int atx_attn_local_prefill(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                           int max_blocks, const int* seq_start, const int* seq_count, const int* seq_pos0, int n_seqs,
                           int total_rows, const float* gate, long long ldg, void* out, long long ldo, int H, int G, int D,
                           int Vd, int block_size, float scale, float softcap, int chunk, int sink, float out_scale,
                           int dtype, int flags, atx_stream_t stream) {
    if (!atx_attn_local_prefill_supported(D, Vd, dtype)) {
        set_error("atx_attn_local_prefill: bf16 with head sizes (64, 64) or (128, 128) only; got D=%d Vd=%d dtype=%d", D, Vd,
                  dtype);
        return ATX_ERR_UNSUPPORTED;
    }
    return atx_attn_window_prefill(q, k_cache, v_cache, D, Vd, block_tables, max_blocks, seq_start, seq_count, seq_pos0,
                                   n_seqs, total_rows, gate, ldg, out, ldo, H, G, D, Vd, block_size, scale, softcap, chunk,
                                   0, nullptr, nullptr, sink, out_scale, dtype, flags, stream);
}

int atx_attn_window_prefill_supported(int D, int Vd, long long k_row, long long v_row, int dtype) {
    return dtype == ATX_DT_BF16 && D > 0 && Vd > 0 && D % 8 == 0 && Vd % 8 == 0 && k_row % 8 == 0 && v_row % 8 == 0 &&
                   tc_key_width(D) && tc_value_width(Vd)
               ? 1
               : 0;
}

int atx_attn_window_prefill(const void* q, const void* k_cache, const void* v_cache, long long k_row, long long v_row,
                            const int* block_tables, int max_blocks, const int* seq_start, const int* seq_count,
                            const int* seq_pos0, int n_seqs, int total_rows, const float* gate, long long ldg, void* out,
                            long long ldo, int H, int G, int D, int Vd, int block_size, float scale, float softcap,
                            int chunk, int window, const float* slopes, const float* sinks, int sink, float out_scale,
                            int dtype, int flags, atx_stream_t stream) {
    const atx_attn_opts o = softmax_opts(scale, softcap, chunk, window, slopes, sinks, sink, out_scale);
    return atx_attn_paged_prefill(q, k_cache, v_cache, k_row, v_row, block_tables, max_blocks, seq_start, seq_count, seq_pos0,
                                  n_seqs, total_rows, gate, ldg, out, ldo, H, G, D, Vd, block_size, &o, dtype, flags, stream);
}

static void fill_tc_args(AttnTcArgs& a, const atx_attn_opts* o) {
    a.slopes = o->slopes, a.sinks = o->sinks, a.bias = o->bias;
    a.chunk = o->chunk, a.window = o->window, a.keep_first = o->keep_first, a.sink = o->sink;
    a.sigmoid_w = o->weight == ATX_ATTN_SIGMOID ? 1 : 0, a.gate_elem = o->gate_elem;
    a.scale = o->scale, a.softcap = o->softcap, a.out_scale = o->out_scale;
}

int atx_attn_paged_prefill(const void* q, const void* k_cache, const void* v_cache, long long k_row, long long v_row,
                           const int* block_tables, int max_blocks, const int* seq_start, const int* seq_count,
                           const int* seq_pos0, int n_seqs, int total_rows, const float* gate, long long ldg, void* out,
                           long long ldo, int H, int G, int D, int Vd, int block_size, const atx_attn_opts* o, int dtype,
                           int flags, atx_stream_t stream) {
    ATX_REQUIRE(q && k_cache && v_cache && block_tables && seq_start && seq_count && seq_pos0 && out,
                "atx_attn_paged_prefill: null pointer");
    ATX_REQUIRE(opts_ok(o), "atx_attn_paged_prefill: bad options");
    ATX_REQUIRE(n_seqs > 0 && total_rows > 0 && H > 0 && G > 0 && H % G == 0 && block_size > 0 && k_row >= D && v_row >= Vd &&
                    ldo % 2 == 0 && (!o->gate_elem || ldg % 2 == 0),
                "atx_attn_paged_prefill: bad shape n_seqs=%d rows=%d H=%d G=%d k_row=%lld v_row=%lld ldo=%lld", n_seqs,
                total_rows, H, G, k_row, v_row, ldo);
    if (!atx_attn_window_prefill_supported(D, Vd, k_row, v_row, dtype) ||
        ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 3)) {
        set_error("atx_attn_paged_prefill: bf16, 16-byte aligned buffers, head and row sizes in multiples of 8, key size "
                  "<= 256 and value size <= 128 only; got D=%d Vd=%d k_row=%lld v_row=%lld dtype=%d", D, Vd, k_row, v_row,
                  dtype);
        return ATX_ERR_UNSUPPORTED;
    }
    AttnTcArgs a = {};
    a.q = q, a.k_cache = k_cache, a.v_cache = v_cache;
    a.block_tables = block_tables, a.seq_start = seq_start, a.seq_count = seq_count, a.seq_pos0 = seq_pos0;
    a.gate = gate, a.out = out;
    a.ldg = ldg, a.ldo = ldo, a.k_row = k_row, a.v_row = v_row;
    a.max_blocks = max_blocks, a.n_seqs = n_seqs;
    a.max_tiles = (total_rows + kTcRows - 1) / kTcRows + n_seqs;   // every sequence adds at most one partly filled tile
    a.H = H, a.G = G, a.D = D, a.Vd = Vd, a.bs = block_size, a.flags = flags;
    fill_tc_args(a, o);
    return dispatch_attn_tc<false>(a, reinterpret_cast<cudaStream_t>(stream));
}

int atx_attn_window_decode_supported(int H, int G, int D, int Vd, long long k_row, long long v_row, int dtype) {
    return G > 0 && H % G == 0 && H / G <= kTcRows && atx_attn_window_prefill_supported(D, Vd, k_row, v_row, dtype) ? 1 : 0;
}

long long atx_attn_window_decode_workspace_bytes(int T, int H, int Vd, int splits) {
    const int vw = tc_value_width(Vd);
    if (T <= 0 || H <= 0 || splits <= 1 || !vw) return 0;
    return static_cast<long long>(T) * H * splits * (vw + 2) * 4;
}

int atx_attn_window_decode(const void* q, const void* k_cache, const void* v_cache, long long k_row, long long v_row,
                           const int* block_tables, int max_blocks, const int* tok_seq, const int* positions,
                           const float* gate, long long ldg, void* out, long long ldo, void* workspace,
                           long long workspace_bytes, int splits, int T, int H, int G, int D, int Vd, int block_size,
                           float scale, float softcap, int chunk, int window, const float* slopes, const float* sinks,
                           int sink, float out_scale, int dtype, int flags, atx_stream_t stream) {
    const atx_attn_opts o = softmax_opts(scale, softcap, chunk, window, slopes, sinks, sink, out_scale);
    return atx_attn_paged_decode(q, k_cache, v_cache, k_row, v_row, block_tables, max_blocks, tok_seq, positions, gate, ldg,
                                 out, ldo, workspace, workspace_bytes, splits, T, H, G, D, Vd, block_size, &o, dtype, flags,
                                 stream);
}

int atx_attn_paged_decode(const void* q, const void* k_cache, const void* v_cache, long long k_row, long long v_row,
                          const int* block_tables, int max_blocks, const int* tok_seq, const int* positions,
                          const float* gate, long long ldg, void* out, long long ldo, void* workspace,
                          long long workspace_bytes, int splits, int T, int H, int G, int D, int Vd, int block_size,
                          const atx_attn_opts* o, int dtype, int flags, atx_stream_t stream) {
    ATX_REQUIRE(q && k_cache && v_cache && block_tables && tok_seq && positions && out, "atx_attn_paged_decode: null pointer");
    ATX_REQUIRE(opts_ok(o), "atx_attn_paged_decode: bad options");
    ATX_REQUIRE(T > 0 && H > 0 && G > 0 && H % G == 0 && block_size > 0 && k_row >= D && v_row >= Vd && ldo % 2 == 0 &&
                    splits >= 1 && splits <= 64 && G <= 65535 && (!o->gate_elem || ldg % 2 == 0),
                "atx_attn_paged_decode: bad shape T=%d H=%d G=%d k_row=%lld v_row=%lld ldo=%lld splits=%d", T, H, G, k_row,
                v_row, ldo, splits);
    if (!atx_attn_window_decode_supported(H, G, D, Vd, k_row, v_row, dtype) ||
        ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 3)) {
        set_error("atx_attn_paged_decode: bf16, 16-byte aligned buffers, sizes in multiples of 8, key size <= 256, value "
                  "size <= 128, at most 64 query heads per key/value head; got H=%d G=%d D=%d Vd=%d dtype=%d", H, G, D, Vd,
                  dtype);
        return ATX_ERR_UNSUPPORTED;
    }
    ATX_REQUIRE(workspace_bytes >= atx_attn_window_decode_workspace_bytes(T, H, Vd, splits) &&
                    (splits == 1 || (workspace && (reinterpret_cast<uintptr_t>(workspace) & 7) == 0)),
                "atx_attn_paged_decode: %d slices need %lld bytes of scratch (8-byte aligned), got %lld", splits,
                atx_attn_window_decode_workspace_bytes(T, H, Vd, splits), workspace_bytes);
    AttnTcArgs a = {};
    a.q = q, a.k_cache = k_cache, a.v_cache = v_cache;
    a.block_tables = block_tables, a.tok_seq = tok_seq, a.positions = positions;
    a.gate = gate, a.out = out;
    a.ldg = ldg, a.ldo = ldo, a.k_row = k_row, a.v_row = v_row;
    a.max_blocks = max_blocks, a.n_seqs = T, a.splits = splits, a.ws = reinterpret_cast<float*>(workspace);
    a.H = H, a.G = G, a.D = D, a.Vd = Vd, a.bs = block_size, a.flags = flags;
    fill_tc_args(a, o);
    return dispatch_attn_tc<true>(a, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
