// Per-head and element-wise operations that sit between a model's projections and its attention kernels:
//   * the element-wise squashing norm  out = tanh(alpha x) w + b  (no row statistics; optional row gather),
//   * a unary activation between the two feed-forward GEMMs (squared ReLU, tanh-GELU),
//   * "head preparation": slices of a fused projection row are cut into heads, each head optionally RMS-normed over its
//     leading elements, rotated in adjacent pairs over a sub-range, blended with the same token's values of an earlier
//     layer, and written either to a row buffer (queries, GEMM inputs) or into the paged cache at the token's slot.
//     A launch takes up to four such slices, so that q, k and v of a layer (or the two bottlenecks of a latent
//     attention) are prepared together,
//   * a small matrix product per head  out[t, h, :] = W_h x[t, h, :]  with an optional sigmoid gate per output element
//     (the per-head up-projections of latent attention in its absorbed form).
// Element type XT (weights, GEMM inputs, pages) = bf16 or fp32; sums, norms, rotations and blends are fp32.
#include "common.cuh"

#include "../../include/atx_b200.h"

namespace atx {

template <typename XT>
__device__ __forceinline__ float hld(const XT* p, long long i);
template <>
__device__ __forceinline__ float hld<float>(const float* p, long long i) {
    return p[i];
}
template <>
__device__ __forceinline__ float hld<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
    return __bfloat162float(p[i]);
}
__device__ __forceinline__ void hst(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void hst(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float4 hld4(const float* p, long long i4) { return reinterpret_cast<const float4*>(p)[i4]; }
__device__ __forceinline__ float4 hld4(const __nv_bfloat16* p, long long i4) {
    const uint2 u = reinterpret_cast<const uint2*>(p)[i4];
    return make_float4(bf16lo(u.x), bf16hi(u.x), bf16lo(u.y), bf16hi(u.y));
}
__device__ __forceinline__ void hst4(float* p, long long i4, float4 v) { reinterpret_cast<float4*>(p)[i4] = v; }
__device__ __forceinline__ void hst4(__nv_bfloat16* p, long long i4, float4 v) {
    reinterpret_cast<uint2*>(p)[i4] = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
}

static void set_pdl_attr(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int flags) {
    if (flags & ATX_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
}

#define ATX_HEADOPS_XT(dtype, ...)       \
    do {                                 \
        if ((dtype) == ATX_DT_F32) {     \
            using XT = float;            \
            __VA_ARGS__;                 \
        } else {                         \
            using XT = __nv_bfloat16;    \
            __VA_ARGS__;                 \
        }                                \
    } while (0)

// ---- tanh norm ---------------------------------------------------------------------------------------------------------
// Blocks [0, T) take one row each; the blocks after them clear zero_ptr (the accumulator of a split-K GEMM that follows).
template <typename XT>
__global__ void __launch_bounds__(256)
tanh_norm_kernel(const float* __restrict__ x, const int* __restrict__ rows, float alpha, const XT* __restrict__ w,
                 const XT* __restrict__ b, XT* __restrict__ out, int T, int W, uint4* __restrict__ zero_ptr,
                 long long zero_vecs) {
    pdl_launch_dependents();
    if (static_cast<int>(blockIdx.x) >= T) {
        pdl_wait();   // a kernel of the previous layer may still be reading the buffer
        const long long nb = gridDim.x - T, b0 = blockIdx.x - T;
        for (long long i = b0 * blockDim.x + threadIdx.x; i < zero_vecs; i += nb * blockDim.x)
            zero_ptr[i] = make_uint4(0, 0, 0, 0);
        return;
    }
    pdl_wait();
    const int t = blockIdx.x;
    const long long r = rows ? rows[t] : t;
    const float* src = x + r * W;
    XT* dst = out + static_cast<long long>(t) * W;
    const bool vec = (W & 3) == 0 && ((reinterpret_cast<unsigned long long>(x) | reinterpret_cast<unsigned long long>(out) |
                                       reinterpret_cast<unsigned long long>(w) | reinterpret_cast<unsigned long long>(b)) & 15) == 0;
    if (vec) {
        for (int i = threadIdx.x; i < W / 4; i += blockDim.x) {
            const float4 v = hld4(src, i), g = hld4(w, i), c = hld4(b, i);
            float4 o;
            o.x = fmaf(tanhf(alpha * v.x), g.x, c.x);
            o.y = fmaf(tanhf(alpha * v.y), g.y, c.y);
            o.z = fmaf(tanhf(alpha * v.z), g.z, c.z);
            o.w = fmaf(tanhf(alpha * v.w), g.w, c.w);
            hst4(dst, i, o);
        }
        return;
    }
    for (int i = threadIdx.x; i < W; i += blockDim.x) hst(dst, i, fmaf(tanhf(alpha * src[i]), hld(w, i), hld(b, i)));
}

// ---- unary activation ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ float unary_act(float z, int kind) {
    if (kind == ATX_ACT_RELU2) {
        const float r = fmaxf(z, 0.f);
        return r * r;
    }
    // tanh form of GELU: z/2 (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
    const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    return 0.5f * z * (1.f + tanhf(u));
}

template <typename XT>
__global__ void __launch_bounds__(256)
unary_act_kernel(const float* __restrict__ in, long long ldi, XT* __restrict__ out, long long ldo, int T, int I, int kind) {
    pdl_launch_dependents();
    pdl_wait();
    const long long n = static_cast<long long>(T) * I;
    for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < n;
         e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long t = e / I;
        const int i = static_cast<int>(e - t * I);
        hst(out, t * ldo + i, unary_act(in[t * ldi + i], kind));
    }
}

// ---- head preparation ----------------------------------------------------------------------------------------------------
struct PrepArgs {
    int n;
    int total_heads;
    atx_head_seg seg[ATX_HEAD_SEGS_MAX];
};

// One warp per (row, head); WIDE: one CTA per (row, head), for steps of few rows whose heads are wide (a bottleneck of
// a thousand elements normed by one warp is a chain of dependent loads). A lane owns single elements (or four); a rotated
// element also reads its partner of the pair.
template <typename XT, bool WIDE>
__global__ void __launch_bounds__(256)
head_prepare_kernel(const float* __restrict__ src, long long ld, const int* __restrict__ positions,
                    const int* __restrict__ slots, int T, int bs, float eps, const __grid_constant__ PrepArgs a) {
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    constexpr int kStep = WIDE ? 256 : 32;
    const int lane = WIDE ? threadIdx.x : (threadIdx.x & 31);
    const long long wid = WIDE ? static_cast<long long>(blockIdx.x)
                               : static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    auto head_sum = [&](float v) -> float {   // over the threads that share the head
        v = warp_sum(v);
        if constexpr (WIDE) {
            if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
            __syncthreads();
            v = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) v += red[i];
        }
        return v;
    };
    if (wid >= static_cast<long long>(T) * a.total_heads) return;
    const long long t = wid / a.total_heads;
    int hh = static_cast<int>(wid - t * a.total_heads);
    int si = 0;
    while (si + 1 < a.n && hh >= a.seg[si].heads) {
        hh -= a.seg[si].heads;
        ++si;
    }
    const atx_head_seg& s = a.seg[si];
    const int slot = slots ? slots[t] : 0;
    if (slot < 0) return;   // padded row
    const float* x = src + t * ld + s.src_off + static_cast<long long>(hh) * s.src_stride;
    const XT* nw = reinterpret_cast<const XT*>(s.norm_w);
    float r = 1.f;
    const float* cs = nullptr;
    const int half = s.rot_dims / 2;
    if (s.rot_dims > 0) cs = s.rot + static_cast<long long>(positions[t]) * s.rot_dims;
    XT* dst;
    if (s.dst_kind == ATX_HEAD_DST_PAGES) {
        const int blk = slot / bs, off = slot - blk * bs;
        dst = reinterpret_cast<XT*>(s.dst) +
              ((static_cast<long long>(blk) * s.heads + hh) * bs + off) * s.dst_stride + s.dst_off;
    } else {
        dst = reinterpret_cast<XT*>(s.dst) + t * s.dst_ld + s.dst_off + static_cast<long long>(hh) * s.dst_stride;
    }
    const long long flat = (t * s.heads + hh) * s.width;   // index into mix_src / save
    // Four elements per access where every offset, pitch and count of the slice is a multiple of four and the pointers
    // are aligned: a rotated pair then lies inside one access, so no partner has to be fetched.
    const bool vec =
        ((s.width | s.src_off | s.src_stride | s.norm_dims | s.rot_off | s.dst_off | s.dst_stride) & 3) == 0 && (ld & 3) == 0 &&
        (s.dst_kind == ATX_HEAD_DST_PAGES || (s.dst_ld & 3) == 0) &&
        ((reinterpret_cast<unsigned long long>(src) | reinterpret_cast<unsigned long long>(s.dst) |
          reinterpret_cast<unsigned long long>(s.norm_w) | reinterpret_cast<unsigned long long>(s.mix_src) |
          reinterpret_cast<unsigned long long>(s.save)) & 15) == 0 &&
        (!s.rot_half || (half & 3) == 0);   // half-split pairs: the partner's four elements are one more aligned access
    if (vec) {
        if (s.norm_dims > 0) {
            float ss = 0.f;
#pragma unroll 4
            for (int i4 = lane; i4 < s.norm_dims / 4; i4 += kStep) {
                const float4 v = hld4(x, i4);
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
            ss = head_sum(ss);
            r = rsqrtf(ss / static_cast<float>(s.norm_dims) + eps);
        }
#pragma unroll 2
        for (int i4 = lane; i4 < s.width / 4; i4 += kStep) {
            const float4 v = hld4(x, i4);
            float e[4] = {v.x, v.y, v.z, v.w};
            const int i = 4 * i4;
            if (i < s.norm_dims) {
                const float4 g = hld4(nw, i4);
                e[0] *= r * g.x, e[1] *= r * g.y, e[2] *= r * g.z, e[3] *= r * g.w;
            }
            if (s.rot_half) {
                // element j < half pairs with j + half: (u, w) -> (u c - w s, w c + u s), angle index j mod half
                const int j = i - s.rot_off;
                if (j >= 0 && j < s.rot_dims) {
                    const bool low = j < half;
                    const int ip4 = low ? i4 + half / 4 : i4 - half / 4;
                    const float4 pv = hld4(x, ip4);
                    float pe[4] = {pv.x, pv.y, pv.z, pv.w};
                    if (4 * ip4 < s.norm_dims) {
                        const float4 g = hld4(nw, ip4);
                        pe[0] *= r * g.x, pe[1] *= r * g.y, pe[2] *= r * g.z, pe[3] *= r * g.w;
                    }
                    const int a0 = low ? j : j - half;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float c = cs[a0 + q], sn = cs[half + a0 + q];
                        e[q] = low ? fmaf(e[q], c, -(pe[q] * sn)) : fmaf(e[q], c, pe[q] * sn);
                    }
                }
            }
#pragma unroll
            for (int p2 = 0; p2 < 2; ++p2) {
                const int j = s.rot_half ? -1 : i + 2 * p2 - s.rot_off;
                if (j >= 0 && j < s.rot_dims) {
                    const float c = cs[j >> 1], sn = cs[half + (j >> 1)];
                    const float a0 = e[2 * p2], b0 = e[2 * p2 + 1];
                    e[2 * p2] = fmaf(a0, c, -(b0 * sn));
                    e[2 * p2 + 1] = fmaf(b0, c, a0 * sn);
                }
            }
            if (s.save) *reinterpret_cast<float4*>(s.save + flat + i) = make_float4(e[0], e[1], e[2], e[3]);
            if (s.mix_src) {
                const float4 mv = *reinterpret_cast<const float4*>(s.mix_src + flat + i);
                e[0] = fmaf(s.mix, mv.x - e[0], e[0]), e[1] = fmaf(s.mix, mv.y - e[1], e[1]);
                e[2] = fmaf(s.mix, mv.z - e[2], e[2]), e[3] = fmaf(s.mix, mv.w - e[3], e[3]);
            }
            hst4(dst, i4, make_float4(e[0], e[1], e[2], e[3]));
        }
        return;
    }
    if (s.norm_dims > 0) {
        float ss = 0.f;
#pragma unroll 4
        for (int i = lane; i < s.norm_dims; i += kStep) ss = fmaf(x[i], x[i], ss);
        ss = head_sum(ss);
        r = rsqrtf(ss / static_cast<float>(s.norm_dims) + eps);
    }
    auto normed = [&](int i) -> float {
        float v = x[i];
        if (i < s.norm_dims) v = v * r * hld(nw, i);
        return v;
    };
    for (int i = lane; i < s.width; i += kStep) {
        float v = normed(i);
        const int j = i - s.rot_off;
        if (j >= 0 && j < s.rot_dims) {
            if (s.rot_half) {
                const bool low = j < half;
                const float p = normed(s.rot_off + (low ? j + half : j - half));
                const int a0 = low ? j : j - half;
                const float c = cs[a0], sn = cs[half + a0];
                v = low ? fmaf(v, c, -(p * sn)) : fmaf(v, c, p * sn);
            } else {
                const float p = normed(s.rot_off + (j ^ 1));
                const float c = cs[j >> 1], sn = cs[half + (j >> 1)];
                // pair (u, w) -> (u c - w s, w c + u s)
                v = (j & 1) ? fmaf(v, c, p * sn) : fmaf(v, c, -(p * sn));
            }
        }
        if (s.save) s.save[flat + i] = v;
        if (s.mix_src) v = fmaf(s.mix, s.mix_src[flat + i] - v, v);   // (1 - mix) v + mix m
        hst(dst, i, v);
    }
}

// ---- per-head matrix product --------------------------------------------------------------------------------------------
// out[t, h * os + n] = (sum_k X[t, x_off + h * xs + k] W[(h N + n) ldw + k]) (* sigmoid(gate[t, h N + n])).
// FMA pipe, fp32 accumulation in a fixed order; 64 x 64 outputs per CTA, 4 x 4 per thread; blockIdx.z = head.
constexpr int kHM = 64, kHN = 64, kHK = 16;

template <typename XT, typename XI>
__global__ void __launch_bounds__(256)
head_gemm_kernel(const XI* __restrict__ X, long long ldx, int x_off, int xs, const XT* __restrict__ W, long long ldw,
                 const float* __restrict__ gate, long long ldg, XT* __restrict__ out, long long ldo, int o_off, int os,
                 int T, int N, int K) {
    __shared__ float sx[kHK][kHM + 1];
    __shared__ float sw[kHK][kHN + 1];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.z;
    const int t0 = blockIdx.y * kHM, n0 = blockIdx.x * kHN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const XI* Xh = X + x_off + static_cast<long long>(h) * xs;
    const XT* Wh = W + static_cast<long long>(h) * N * ldw;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += kHK) {
        for (int e = threadIdx.x; e < kHM * kHK; e += 256) {
            const int rr = e / kHK, kk = e - rr * kHK;
            const int t = t0 + rr, k = k0 + kk, n = n0 + rr;
            sx[kk][rr] = (t < T && k < K) ? hld(Xh, static_cast<long long>(t) * ldx + k) : 0.f;
            sw[kk][rr] = (n < N && k < K) ? hld(Wh, static_cast<long long>(n) * ldw + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kHK; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = sx[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = sw[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + ty * 4 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (gate) v *= 1.f / (1.f + expf(-gate[static_cast<long long>(t) * ldg + static_cast<long long>(h) * N + n]));
            hst(out, static_cast<long long>(t) * ldo + o_off + static_cast<long long>(h) * os + n, v);
        }
    }
}

// The same product on the tensor cores (bf16 operands, fp32 accumulation): 64 rows x 64 outputs of one head per CTA, a
// warp owns 16 rows; X (fp32 or bf16) and W are staged as bf16 in chunks of 64 reduction elements, zero past the edges.
constexpr int kHT = 64, kHKC = 64, kHLD = kHKC + 8;

template <typename XI>
__global__ void __launch_bounds__(128)
head_gemm_tc_kernel(const XI* __restrict__ X, long long ldx, int x_off, int xs, const __nv_bfloat16* __restrict__ W,
                    long long ldw, const float* __restrict__ gate, long long ldg, __nv_bfloat16* __restrict__ out,
                    long long ldo, int o_off, int os, int T, int N, int K) {
    __shared__ __align__(16) __nv_bfloat16 sx[kHT * kHLD];
    __shared__ __align__(16) __nv_bfloat16 sw[kHT * kHLD];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.z;
    const int t0 = blockIdx.y * kHT, n0 = blockIdx.x * kHT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const XI* Xh = X + x_off + static_cast<long long>(h) * xs;
    const __nv_bfloat16* Wh = W + static_cast<long long>(h) * N * ldw;
    float acc[kHT / 8][4];
#pragma unroll
    for (int i = 0; i < kHT / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    // eight elements per access where pitches, offsets and K allow it (rows past T or N and columns past K stay zero)
    const bool vec = ((K | x_off | xs) & 7) == 0 && ((ldx | ldw) & 7) == 0 &&
                     ((reinterpret_cast<unsigned long long>(X) | reinterpret_cast<unsigned long long>(W)) & 15) == 0;
    for (int k0 = 0; k0 < K; k0 += kHKC) {
        if (vec) {
            for (int e = threadIdx.x; e < kHT * (kHKC / 8); e += 128) {
                const int r = e / (kHKC / 8), k8 = (e - r * (kHKC / 8)) * 8;
                const int t = t0 + r, n = n0 + r, k = k0 + k8;
                uint4 xv = make_uint4(0, 0, 0, 0), wv = make_uint4(0, 0, 0, 0);
                if (t < T && k < K) {
                    if constexpr (sizeof(XI) == 4) {
                        const float4 a = *reinterpret_cast<const float4*>(Xh + static_cast<long long>(t) * ldx + k);
                        const float4 b = *reinterpret_cast<const float4*>(Xh + static_cast<long long>(t) * ldx + k + 4);
                        xv = make_uint4(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w), pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
                    } else {
                        xv = *reinterpret_cast<const uint4*>(Xh + static_cast<long long>(t) * ldx + k);
                    }
                }
                if (n < N && k < K) wv = __ldg(reinterpret_cast<const uint4*>(Wh + static_cast<long long>(n) * ldw + k));
                *reinterpret_cast<uint4*>(sx + r * kHLD + k8) = xv;
                *reinterpret_cast<uint4*>(sw + r * kHLD + k8) = wv;
            }
        } else {
            for (int e = threadIdx.x; e < kHT * kHKC; e += 128) {
                const int r = e / kHKC, kk = e - r * kHKC;
                const int t = t0 + r, n = n0 + r, k = k0 + kk;
                const float xv = (t < T && k < K) ? hld(Xh, static_cast<long long>(t) * ldx + k) : 0.f;
                sx[r * kHLD + kk] = __float2bfloat16_rn(xv);
                sw[r * kHLD + kk] = (n < N && k < K) ? Wh[static_cast<long long>(n) * ldw + k] : __float2bfloat16_rn(0.f);
            }
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < kHKC / 16; ++ks) {
            uint32_t a[4];
            ldsm_x4(smem_u32(sx + (warp * 16 + (lane & 15)) * kHLD + ks * 16 + (lane >> 4) * 8), a[0], a[1], a[2], a[3]);
#pragma unroll
            for (int nb2 = 0; nb2 < kHT / 16; ++nb2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(smem_u32(sw + (nb2 * 16 + (lane >> 4) * 8 + (lane & 7)) * kHLD + ks * 16 + ((lane >> 3) & 1) * 8), b0,
                        b1, b2, b3);
                mma_bf16(acc[2 * nb2], a, b0, b1);
                mma_bf16(acc[2 * nb2 + 1], a, b2, b3);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int t = t0 + warp * 16 + (lane >> 2) + 8 * rr;
        if (t >= T) continue;
#pragma unroll
        for (int nb = 0; nb < kHT / 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int n = n0 + nb * 8 + (lane & 3) * 2 + e;
                if (n >= N) continue;
                float v = acc[nb][2 * rr + e];
                if (gate) v *= 1.f / (1.f + __expf(-gate[static_cast<long long>(t) * ldg + static_cast<long long>(h) * N + n]));
                out[static_cast<long long>(t) * ldo + o_off + static_cast<long long>(h) * os + n] = __float2bfloat16_rn(v);
            }
        }
    }
}

}  // namespace atx

using namespace atx;

extern "C" {

int atx_tanh_norm(const float* x, const int* rows, float alpha, const void* w, const void* b, void* out, int T, int W,
                  void* zero_ptr, long long zero_bytes, int dtype, int flags, atx_stream_t stream) {
    ATX_REQUIRE(x && w && b && out, "atx_tanh_norm: null pointer");
    ATX_REQUIRE(T > 0 && W > 0, "atx_tanh_norm: bad shape T=%d W=%d", T, W);
    ATX_REQUIRE(zero_bytes >= 0 && zero_bytes % 16 == 0 && (zero_bytes == 0 || zero_ptr),
                "atx_tanh_norm: zero_bytes=%lld must be a non-negative multiple of 16 with a buffer", zero_bytes);
    const long long zv = zero_bytes / 16;
    long long zb = (zv + 256 * 8 - 1) / (256 * 8);
    if (zb > 2048) zb = 2048;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(static_cast<unsigned>(T + zb));
    cfg.blockDim = dim3(256);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl_attr(cfg, attr, flags);
    ATX_HEADOPS_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(&cfg, tanh_norm_kernel<XT>, x, rows, alpha,
                                                      reinterpret_cast<const XT*>(w), reinterpret_cast<const XT*>(b),
                                                      reinterpret_cast<XT*>(out), T, W,
                                                      reinterpret_cast<uint4*>(zero_ptr), zv)));
    return ATX_OK;
}

int atx_unary_act(const float* in, long long ldi, void* out, long long ldo, int T, int I, int kind, int dtype, int flags,
                  atx_stream_t stream) {
    ATX_REQUIRE(in && out, "atx_unary_act: null pointer");
    ATX_REQUIRE(T > 0 && I > 0 && ldi >= I && ldo >= I, "atx_unary_act: bad shape T=%d I=%d ldi=%lld ldo=%lld", T, I, ldi, ldo);
    ATX_REQUIRE(kind == ATX_ACT_RELU2 || kind == ATX_ACT_GELU_TANH, "atx_unary_act: unknown activation %d", kind);
    const long long n = static_cast<long long>(T) * I;
    long long blocks = (n + 256 * 4 - 1) / (256 * 4);
    if (blocks > 148 * 16) blocks = 148 * 16;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(static_cast<unsigned>(blocks));
    cfg.blockDim = dim3(256);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl_attr(cfg, attr, flags);
    ATX_HEADOPS_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(&cfg, unary_act_kernel<XT>, in, ldi, reinterpret_cast<XT*>(out), ldo,
                                                      T, I, kind)));
    return ATX_OK;
}

int atx_head_prepare(const float* src, long long ld, const atx_head_seg* segs, int n_segs, const int* positions,
                     const int* slots, int T, int block_size, float eps, int dtype, int flags, atx_stream_t stream) {
    ATX_REQUIRE(src && segs, "atx_head_prepare: null pointer");
    ATX_REQUIRE(T > 0 && n_segs > 0 && n_segs <= ATX_HEAD_SEGS_MAX, "atx_head_prepare: T=%d, %d segments (1..%d)", T,
                n_segs, ATX_HEAD_SEGS_MAX);
    PrepArgs a = {};
    a.n = n_segs;
    for (int i = 0; i < n_segs; ++i) {
        const atx_head_seg& s = segs[i];
        ATX_REQUIRE(s.heads > 0 && s.width > 0 && s.dst && s.src_off >= 0 && s.dst_off >= 0,
                    "atx_head_prepare: segment %d: heads=%d width=%d", i, s.heads, s.width);
        ATX_REQUIRE(s.norm_dims >= 0 && s.norm_dims <= s.width && (s.norm_dims == 0 || s.norm_w),
                    "atx_head_prepare: segment %d: norm over %d of %d elements needs a weight", i, s.norm_dims, s.width);
        ATX_REQUIRE(s.rot_dims >= 0 && s.rot_dims % 2 == 0 && s.rot_off >= 0 && s.rot_off + s.rot_dims <= s.width &&
                        (s.rot_dims == 0 || (s.rot && positions)),
                    "atx_head_prepare: segment %d: rotation of [%d, %d) in a head of %d needs an even count, a table and "
                    "positions", i, s.rot_off, s.rot_off + s.rot_dims, s.width);
        ATX_REQUIRE(s.dst_kind == ATX_HEAD_DST_ROWS || (s.dst_kind == ATX_HEAD_DST_PAGES && slots && block_size > 0),
                    "atx_head_prepare: segment %d: pages need slots and a block size", i);
        a.seg[i] = s;
        a.total_heads += s.heads;
    }
    const long long warps = static_cast<long long>(T) * a.total_heads;
    int widest = 0;
    for (int i = 0; i < n_segs; ++i) widest = segs[i].width > widest ? segs[i].width : widest;
    const bool wide = widest >= 512 && warps <= 1024;   // few, wide heads: a CTA each
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(static_cast<unsigned>(wide ? warps : (warps + 7) / 8));
    cfg.blockDim = dim3(256);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl_attr(cfg, attr, flags);
    if (wide)
        ATX_HEADOPS_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(&cfg, head_prepare_kernel<XT, true>, src, ld, positions, slots, T,
                                                          block_size, eps, a)));
    else
        ATX_HEADOPS_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(&cfg, head_prepare_kernel<XT, false>, src, ld, positions, slots, T,
                                                          block_size, eps, a)));
    return ATX_OK;
}

int atx_head_gemm(const void* X, int x_f32, long long ldx, int x_off, int x_head_stride, const void* W, long long ldw,
                  const float* gate, long long ldg, void* out, long long ldo, int o_off, int o_head_stride, int T,
                  int heads, int N, int K, int dtype, int flags, atx_stream_t stream) {
    ATX_REQUIRE(X && W && out, "atx_head_gemm: null pointer");
    ATX_REQUIRE(T > 0 && heads > 0 && heads <= 65535 && N > 0 && K > 0 && ldw >= K,
                "atx_head_gemm: bad shape T=%d heads=%d N=%d K=%d ldw=%lld", T, heads, N, K, ldw);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3((N + kHN - 1) / kHN, (T + kHM - 1) / kHM, heads);
    cfg.blockDim = dim3(256);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl_attr(cfg, attr, flags);
    if (dtype == ATX_DT_BF16 && !(flags & ATX_FLAG_HEAD_GEMM_FMA)) {   // bf16: the tensor cores
        using B = __nv_bfloat16;
        cfg.gridDim = dim3((N + kHT - 1) / kHT, (T + kHT - 1) / kHT, heads);
        cfg.blockDim = dim3(128);
        if (x_f32)
            ATX_CUDA(cudaLaunchKernelEx(&cfg, head_gemm_tc_kernel<float>, reinterpret_cast<const float*>(X), ldx, x_off,
                                        x_head_stride, reinterpret_cast<const B*>(W), ldw, gate, ldg,
                                        reinterpret_cast<B*>(out), ldo, o_off, o_head_stride, T, N, K));
        else
            ATX_CUDA(cudaLaunchKernelEx(&cfg, head_gemm_tc_kernel<B>, reinterpret_cast<const B*>(X), ldx, x_off,
                                        x_head_stride, reinterpret_cast<const B*>(W), ldw, gate, ldg,
                                        reinterpret_cast<B*>(out), ldo, o_off, o_head_stride, T, N, K));
        return ATX_OK;
    }
    if (x_f32 || dtype == ATX_DT_F32) {
        ATX_HEADOPS_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(&cfg, head_gemm_kernel<XT, float>,
                                                          reinterpret_cast<const float*>(X), ldx, x_off, x_head_stride,
                                                          reinterpret_cast<const XT*>(W), ldw, gate, ldg,
                                                          reinterpret_cast<XT*>(out), ldo, o_off, o_head_stride, T, N, K)));
    } else {
        using B = __nv_bfloat16;
        ATX_CUDA(cudaLaunchKernelEx(&cfg, head_gemm_kernel<B, B>, reinterpret_cast<const B*>(X), ldx, x_off, x_head_stride,
                                    reinterpret_cast<const B*>(W), ldw, gate, ldg, reinterpret_cast<B*>(out), ldo, o_off,
                                    o_head_stride, T, N, K));
    }
    return ATX_OK;
}

}  // extern "C"
