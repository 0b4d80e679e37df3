// Row kernels in which a token reads its predecessor, and a feed-forward activation with row statistics:
//   * embedding rows plus a row of a second table chosen by a hash of (previous token, token),
//   * token shift: the normed row blended with the previous position's normed row, per channel,
//   * a polynomial of unit-rms powers of the feed-forward's hidden row.
// The predecessor of a step's first row comes from the sequence's state slot (the last token id; the last normed row of
// every layer), which the CTA that read it then overwrites with the step's last row: reader and writer are the same
// threads, so no second launch is needed. A sequence at position 0 has no predecessor whatever its slot holds.
// A step is a flat batch of rows; sequence s owns rows [seq_start[s], seq_start[s] + seq_count[s]), first position
// seq_pos0[s], state slot seq_slot[s]; tok_seq[t] is the sequence of row t (-1: padded row, skipped).
#include "common.cuh"

#include "../../include/atx_b200.h"

namespace atx {

template <typename XT>
__device__ __forceinline__ float rld(const XT* p, long long i);
template <>
__device__ __forceinline__ float rld<float>(const float* p, long long i) {
    return p[i];
}
template <>
__device__ __forceinline__ float rld<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
    return __bfloat162float(p[i]);
}
__device__ __forceinline__ void rst(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void rst(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }
__device__ __forceinline__ float4 rld4(const float* p, long long i4) { return reinterpret_cast<const float4*>(p)[i4]; }
__device__ __forceinline__ float4 rld4(const __nv_bfloat16* p, long long i4) {
    const uint2 u = reinterpret_cast<const uint2*>(p)[i4];
    return make_float4(bf16lo(u.x), bf16hi(u.x), bf16lo(u.y), bf16hi(u.y));
}
__device__ __forceinline__ void rst4(float* p, long long i4, float4 v) { reinterpret_cast<float4*>(p)[i4] = v; }
__device__ __forceinline__ void rst4(__nv_bfloat16* p, long long i4, float4 v) {
    reinterpret_cast<uint2*>(p)[i4] = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
}

static void set_pdl_row(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int flags) {
    if (flags & ATX_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
}

#define ATX_ROW_XT(dtype_, ...)                \
    do {                                       \
        if ((dtype_) == ATX_DT_F32) {          \
            using XT = float;                  \
            __VA_ARGS__;                       \
        } else {                               \
            using XT = __nv_bfloat16;          \
            __VA_ARGS__;                       \
        }                                      \
    } while (0)

// ---- embedding row + pair-table row -----------------------------------------------------------------------------------
// out[t] = table[id_t] * scale + pair[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets]; a sequence's first token takes
// row `buckets` (the table has buckets + 1 rows). prev_tok [slots]: the last token of every live sequence.
template <typename XT>
__global__ void __launch_bounds__(128)
embed_rows_pair_kernel(const int* __restrict__ ids, const XT* __restrict__ table, float scale, const XT* __restrict__ pair,
                       int buckets, int mul_prev, int mul_cur, int* __restrict__ prev_tok, const int* __restrict__ tok_seq,
                       const int* __restrict__ seq_start, const int* __restrict__ seq_count,
                       const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot, float* __restrict__ out, int W,
                       int V) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int s = tok_seq[t];
    float* dst = out + static_cast<long long>(t) * W;
    if (s < 0) {   // padded row: defined contents, no state
        for (int i = threadIdx.x; i < W; i += blockDim.x) dst[i] = 0.f;
        return;
    }
    auto clamp = [V](int id) { return id < 0 ? 0 : (id >= V ? V - 1 : id); };
    const int id = clamp(ids[t]);
    const int r0 = seq_start[s];
    long long prow = buckets;
    if (t != r0) {
        prow = (static_cast<long long>(clamp(ids[t - 1])) * mul_prev + static_cast<long long>(id) * mul_cur) % buckets;
    } else {
        const int slot = seq_slot[s];
        if (seq_pos0[s] > 0)
            prow = (static_cast<long long>(clamp(prev_tok[slot])) * mul_prev + static_cast<long long>(id) * mul_cur) % buckets;
        __syncthreads();   // every thread has read the slot
        if (threadIdx.x == 0) prev_tok[slot] = ids[r0 + seq_count[s] - 1];
    }
    const XT* src = table + static_cast<long long>(id) * W;
    const XT* ps = pair + prow * W;
    if ((W & 3) == 0 && ((reinterpret_cast<unsigned long long>(table) | reinterpret_cast<unsigned long long>(pair) |
                          reinterpret_cast<unsigned long long>(out)) & 15) == 0) {
#pragma unroll 4
        for (int i = threadIdx.x; i < W / 4; i += blockDim.x) {
            const float4 a = rld4(src, i), b = rld4(ps, i);
            rst4(dst, i, make_float4(fmaf(a.x, scale, b.x), fmaf(a.y, scale, b.y), fmaf(a.z, scale, b.z), fmaf(a.w, scale, b.w)));
        }
        return;
    }
    for (int i = threadIdx.x; i < W; i += blockDim.x) dst[i] = fmaf(rld(src, i), scale, rld(ps, i));
}

// ---- token shift ----------------------------------------------------------------------------------------------------------
// out[t] = x[t] + (x[t-1] - x[t]) * mu, x fp32 (the normed rows), out of the element type; state [slots, W] fp32 keeps
// the last x of every live sequence.
template <typename XT>
__global__ void __launch_bounds__(256)
token_shift_kernel(const float* __restrict__ x, const XT* __restrict__ mu, float* __restrict__ state,
                   const int* __restrict__ tok_seq, const int* __restrict__ seq_start, const int* __restrict__ seq_count,
                   const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot, XT* __restrict__ out, int W) {
    pdl_launch_dependents();
    pdl_wait();
    const long long t = blockIdx.x;
    const int s = tok_seq[t];
    XT* o = out + t * W;
    if (s < 0) {
        for (int i = threadIdx.x; i < W; i += blockDim.x) rst(o, i, 0.f);
        return;
    }
    const int r0 = seq_start[s];
    const bool first = t == r0;
    const bool none = first && seq_pos0[s] == 0;
    const float* cur = x + t * W;
    const float* prev = first ? state + static_cast<long long>(seq_slot[s]) * W : cur - W;
    float* keep = first ? state + static_cast<long long>(seq_slot[s]) * W : nullptr;
    const float* last = x + (static_cast<long long>(r0) + seq_count[s] - 1) * W;   // the step's last row of the sequence
    if ((W & 3) == 0 && ((reinterpret_cast<unsigned long long>(x) | reinterpret_cast<unsigned long long>(mu) |
                          reinterpret_cast<unsigned long long>(state) | reinterpret_cast<unsigned long long>(out)) & 15) == 0) {
#pragma unroll 2
        for (int i = threadIdx.x; i < W / 4; i += blockDim.x) {
            const float4 c = rld4(cur, i), m = rld4(mu, i);
            const float4 p = none ? make_float4(0.f, 0.f, 0.f, 0.f) : rld4(prev, i);
            rst4(o, i, make_float4(fmaf(p.x - c.x, m.x, c.x), fmaf(p.y - c.y, m.y, c.y), fmaf(p.z - c.z, m.z, c.z),
                                   fmaf(p.w - c.w, m.w, c.w)));
            if (keep) rst4(keep, i, rld4(last, i));   // the same thread read this part of the slot above
        }
        return;
    }
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float c = cur[i], p = none ? 0.f : prev[i];
        rst(o, i, fmaf(p - c, rld(mu, i), c));
        if (keep) keep[i] = last[i];
    }
}

// ---- polynomial of unit-rms powers -------------------------------------------------------------------------------------------
// out = a z / rms(z) + b z^2 / rms(z^2) + c z^3 / rms(z^3) + e over a row of F elements; coef = {a, b, c, e} fp32.
template <typename XT>
__global__ void __launch_bounds__(256)
poly_norm_act_kernel(const float* __restrict__ z, long long ldz, const float* __restrict__ coef, XT* __restrict__ out,
                     long long ldo, int F, float eps) {
    __shared__ float red[3][8];
    pdl_launch_dependents();
    const float a = coef[0], b = coef[1], c = coef[2], e = coef[3];
    pdl_wait();
    const long long t = blockIdx.x;
    const float* zr = z + t * ldz;
    XT* o = out + t * ldo;
    const bool vec = (F & 3) == 0 && (ldz & 3) == 0 && (ldo & 3) == 0 &&
                     ((reinterpret_cast<unsigned long long>(z) | reinterpret_cast<unsigned long long>(out)) & 15) == 0;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    auto take = [&](float v) {
        const float v2 = v * v;
        s2 += v2;
        s4 = fmaf(v2, v2, s4);
        s6 = fmaf(v2 * v2, v2, s6);
    };
    if (vec) {
        for (int i = threadIdx.x; i < F / 4; i += blockDim.x) {
            const float4 v = rld4(zr, i);
            take(v.x), take(v.y), take(v.z), take(v.w);
        }
    } else {
        for (int i = threadIdx.x; i < F; i += blockDim.x) take(zr[i]);
    }
    s2 = warp_sum(s2), s4 = warp_sum(s4), s6 = warp_sum(s6);
    if ((threadIdx.x & 31) == 0) {
        red[0][threadIdx.x >> 5] = s2;
        red[1][threadIdx.x >> 5] = s4;
        red[2][threadIdx.x >> 5] = s6;
    }
    __syncthreads();
    s2 = s4 = s6 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s2 += red[0][i], s4 += red[1][i], s6 += red[2][i];
    const float inv = 1.f / static_cast<float>(F);
    const float r1 = a * rsqrtf(s2 * inv + eps), r2 = b * rsqrtf(s4 * inv + eps), r3 = c * rsqrtf(s6 * inv + eps);
    auto act = [&](float v) { return fmaf(v, fmaf(v, fmaf(v, r3, r2), r1), e); };   // ((r3 v + r2) v + r1) v + e
    if (vec) {
        for (int i = threadIdx.x; i < F / 4; i += blockDim.x) {
            const float4 v = rld4(zr, i);
            rst4(o, i, make_float4(act(v.x), act(v.y), act(v.z), act(v.w)));
        }
    } else {
        for (int i = threadIdx.x; i < F; i += blockDim.x) rst(o, i, act(zr[i]));
    }
}

}  // namespace atx

using namespace atx;

extern "C" {

int atx_embed_rows_pair(const int* ids, const void* table, float scale, const void* pair_table, int buckets, int mul_prev,
                        int mul_cur, int* prev_tok, const int* tok_seq, const int* seq_start, const int* seq_count,
                        const int* seq_pos0, const int* seq_slot, float* out, int T, int W, int V, int dtype, int flags,
                        atx_stream_t stream) {
    ATX_REQUIRE(ids && table && pair_table && prev_tok && tok_seq && seq_start && seq_count && seq_pos0 && seq_slot && out,
                "atx_embed_rows_pair: null pointer");
    ATX_REQUIRE(T > 0 && W > 0 && V > 0 && buckets > 0, "atx_embed_rows_pair: bad shape T=%d W=%d V=%d buckets=%d", T, W, V,
                buckets);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(T);
    cfg.blockDim = dim3(128);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl_row(cfg, attr, flags);
    ATX_ROW_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(&cfg, embed_rows_pair_kernel<XT>, ids, reinterpret_cast<const XT*>(table),
                                                  scale, reinterpret_cast<const XT*>(pair_table), buckets, mul_prev, mul_cur,
                                                  prev_tok, tok_seq, seq_start, seq_count, seq_pos0, seq_slot, out, W, V)));
    return ATX_OK;
}

int atx_token_shift(const float* x, const void* mu, float* state, const int* tok_seq, const int* seq_start,
                    const int* seq_count, const int* seq_pos0, const int* seq_slot, void* out, int T, int W, int dtype,
                    int flags, atx_stream_t stream) {
    ATX_REQUIRE(x && mu && state && tok_seq && seq_start && seq_count && seq_pos0 && seq_slot && out,
                "atx_token_shift: null pointer");
    ATX_REQUIRE(T > 0 && W > 0, "atx_token_shift: bad shape T=%d W=%d", T, W);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(T);
    cfg.blockDim = dim3(256);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl_row(cfg, attr, flags);
    ATX_ROW_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(&cfg, token_shift_kernel<XT>, x, reinterpret_cast<const XT*>(mu), state,
                                                  tok_seq, seq_start, seq_count, seq_pos0, seq_slot,
                                                  reinterpret_cast<XT*>(out), W)));
    return ATX_OK;
}

int atx_poly_norm_act(const float* z, long long ldz, const float* coef, void* out, long long ldo, int T, int F, float eps,
                      int dtype, int flags, atx_stream_t stream) {
    ATX_REQUIRE(z && coef && out, "atx_poly_norm_act: null pointer");
    ATX_REQUIRE(T > 0 && F > 0 && ldz >= F && ldo >= F, "atx_poly_norm_act: bad shape T=%d F=%d ldz=%lld ldo=%lld", T, F, ldz,
                ldo);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(T);
    cfg.blockDim = dim3(256);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl_row(cfg, attr, flags);
    ATX_ROW_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(&cfg, poly_norm_act_kernel<XT>, z, ldz, coef, reinterpret_cast<XT*>(out), ldo,
                                                  F, eps)));
    return ATX_OK;
}

}  // extern "C"
