// Kernels of the sequence mixers that carry a recurrent state, and the glue around them:
//   * residual update with a norm on both sides of the sublayer (post-norm of the sublayer's output, add, pre-norm of
//     the next sublayer's input) in one pass over the row,
//   * the decayed outer-product recurrence  S_t = a_t S_(t-1) + (c_t k_t) v_t^T,  y_t = S_t^T q_t (+ d v_t)  that both
//     linear attention with a fixed decay per head and the selective state-space scan are instances of,
//   * the short causal convolution with its carried inputs, the step size / decay of the selective scan,
//   * gated RMS norms of mixer outputs (gate before or after the norm, norm in equal groups),
//   * gate * up activation, embedding rows, [x ; x0] concatenation for a re-entrant block of layers.
// Activations that feed a GEMM (and weights) are `XT` = bf16 or fp32; everything else is fp32. States are fp32.
// A step is a flat batch of rows; sequence s owns rows [seq_start[s], seq_start[s] + seq_count[s]) whose first row is
// position seq_pos0[s]; its states live in slot seq_slot[s]. A sequence at position 0 starts from zero state without
// the slot being cleared first (slots are reused). seq_count 0 marks a padded entry.
#include "common.cuh"

#include "../../include/atx_b200.h"

namespace atx {

template <typename XT>
__device__ __forceinline__ float ldf(const XT* p, long long i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, long long i) {
    return p[i];
}
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
    return __bfloat162float(p[i]);
}
__device__ __forceinline__ void stf(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

// four consecutive elements at element index 4 * i4 (16-byte / 8-byte aligned by the caller's choice of the vector path)
__device__ __forceinline__ float4 ld4(const float* p, long long i4) { return reinterpret_cast<const float4*>(p)[i4]; }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p, long long i4) {
    const uint2 u = reinterpret_cast<const uint2*>(p)[i4];
    return make_float4(bf16lo(u.x), bf16hi(u.x), bf16lo(u.y), bf16hi(u.y));
}
__device__ __forceinline__ void st4(float* p, long long i4, float4 v) { reinterpret_cast<float4*>(p)[i4] = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, long long i4, float4 v) {
    reinterpret_cast<uint2*>(p)[i4] = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

static void set_pdl2(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int flags) {
    if (flags & ATX_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
}

// block-wide sum; every thread gets the result. red: >= 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();  // red may still be read from a previous call
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
    const int nw = (blockDim.x + 31) >> 5;
    for (int i = 0; i < nw; ++i) t += red[i];
    return t;
}

// ---- embedding rows -------------------------------------------------------------------------------------------
template <typename XT>
__global__ void __launch_bounds__(128) embed_rows_kernel(const int* __restrict__ ids, const XT* __restrict__ table,
                                                         float* __restrict__ out, int W, int V, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    const XT* src = table + static_cast<long long>(id) * W;
    float* dst = out + static_cast<long long>(t) * W;
    if ((W & 3) == 0 && ((reinterpret_cast<unsigned long long>(table) | reinterpret_cast<unsigned long long>(out)) & 15) == 0) {
#pragma unroll 4
        for (int i = threadIdx.x; i < W / 4; i += blockDim.x) {  // four elements per access
            float4 v = ld4(src, i);
            v.x *= scale, v.y *= scale, v.z *= scale, v.w *= scale;   // scale 1 leaves the row as it is stored
            st4(dst, i, v);
        }
        return;
    }
    for (int i = threadIdx.x; i < W; i += blockDim.x) dst[i] = ldf(src, i) * scale;
}

// ---- [x ; x0]: the input of the projection that re-enters a block of layers ---------------------------------------
template <typename XT>
__global__ void __launch_bounds__(128) concat_embed_kernel(const float* __restrict__ h, const int* __restrict__ ids,
                                                           const XT* __restrict__ table, XT* __restrict__ out, int W,
                                                           int V) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    XT* o = out + static_cast<long long>(t) * 2 * W;
    if ((W & 3) == 0 && ((reinterpret_cast<unsigned long long>(table) | reinterpret_cast<unsigned long long>(out) |
                          reinterpret_cast<unsigned long long>(h)) & 15) == 0) {
        const float* hr = h + static_cast<long long>(t) * W;
        const XT* src = table + static_cast<long long>(id) * W;
#pragma unroll 4
        for (int i = threadIdx.x; i < W / 4; i += blockDim.x) {  // four elements per access
            st4(o, i, ld4(hr, i));
            st4(o + W, i, ld4(src, i));
        }
        return;
    }
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        stf(o, i, h[static_cast<long long>(t) * W + i]);
        o[W + i] = table[static_cast<long long>(id) * W + i];
    }
}

// ---- residual update between two norms ---------------------------------------------------------------------------
// h[r] += rms(y[r]) * w_post (if y) + vec (if vec);  out[t] = rms(h[r]) * w_pre (if w_pre);  r = rows ? rows[t] : t.
// With `rows` the residual itself is left untouched (the gathered rows feed the LM head only).
// zero_y: the row of y is cleared once it has been read, so that the next split-K GEMM can accumulate into it;
// CTAs beyond T clear zero_ptr (the accumulator of the GEMM that consumes `out`).
// post_scale (nullable): a second weight vector on the post-normed sublayer output (a learned scale per channel of the
// residual branch). OT: the element type of `out`, XT or fp32 (a consumer that still works on the normed row in fp32).
template <typename XT, typename OT, bool VEC>
__global__ void __launch_bounds__(1024)
resid_norm_kernel(float* __restrict__ h, float* __restrict__ y, const XT* __restrict__ w_post,
                  const XT* __restrict__ post_scale, const XT* __restrict__ vec, const XT* __restrict__ w_pre,
                  OT* __restrict__ out, const int* __restrict__ rows, int T, int W, float eps, int zero_y,
                  uint4* __restrict__ zero_ptr, long long zero_vecs, float out_scale) {
    extern __shared__ __align__(16) float srow[];
    __shared__ float red[32];
    pdl_launch_dependents();
    // One vector per thread covers the row (few rows, many threads): everything stays in registers, and the weights,
    // which no kernel writes, are fetched before the wait for the producer of h and y.
    const bool in_regs = VEC && W / 4 <= static_cast<int>(blockDim.x);
    const bool on = in_regs && static_cast<int>(threadIdx.x) < W / 4 && static_cast<int>(blockIdx.x) < T;
    float4 wp4 = make_float4(0.f, 0.f, 0.f, 0.f), vc4 = wp4, wq4 = wp4;
    if (VEC && on) {
        if (w_post) wp4 = ld4(w_post, threadIdx.x);
        if (post_scale) {
            const float4 l4 = ld4(post_scale, threadIdx.x);
            wp4.x *= l4.x, wp4.y *= l4.y, wp4.z *= l4.z, wp4.w *= l4.w;
        }
        if (vec) vc4 = ld4(vec, threadIdx.x);
        if (w_pre) wq4 = ld4(w_pre, threadIdx.x);
    }
    pdl_wait();
    if (blockIdx.x >= T) {
        const long long nb = gridDim.x - T;
        for (long long i = static_cast<long long>(blockIdx.x - T) * blockDim.x + threadIdx.x; i < zero_vecs;
             i += nb * blockDim.x)
            zero_ptr[i] = make_uint4(0, 0, 0, 0);
        return;
    }
    const int t = blockIdx.x;
    const long long r = rows ? rows[t] : t;
    float* hr = h + r * W;
    float rs_y = 0.f;
    if (VEC && in_regs) {
        const int i = threadIdx.x;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f), a = v;
        if (on) {
            v = ld4(hr, i);
            if (y) {
                a = ld4(y + r * W, i);
                if (zero_y) st4(y + r * W, i, make_float4(0.f, 0.f, 0.f, 0.f));
            }
        }
        if (y) {
            rs_y = rsqrtf(block_sum(a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w, red) / static_cast<float>(W) + eps);
            v.x += a.x * rs_y * wp4.x, v.y += a.y * rs_y * wp4.y, v.z += a.z * rs_y * wp4.z, v.w += a.w * rs_y * wp4.w;
        }
        v.x += vc4.x, v.y += vc4.y, v.z += vc4.z, v.w += vc4.w;
        if (on && (y || vec) && !rows) st4(hr, i, v);
        if (!out) return;
        if (!w_pre) {   // no norm in front of the consumer: the row itself in the element type
            if (on) st4(out + static_cast<long long>(t) * W, i, make_float4(v.x * out_scale, v.y * out_scale, v.z * out_scale, v.w * out_scale));
            return;
        }
        const float rs = rsqrtf(block_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w, red) / static_cast<float>(W) + eps) * out_scale;
        if (on) st4(out + static_cast<long long>(t) * W, i, make_float4(v.x * rs * wq4.x, v.y * rs * wq4.y, v.z * rs * wq4.z, v.w * rs * wq4.w));
        return;
    }
    if (VEC) {   // W a multiple of 4 and every row 16-byte aligned (8 for bf16): four elements per load and store
        const int W4 = W / 4;
        float4* srow4 = reinterpret_cast<float4*>(srow);
        if (y) {
            float ss = 0.f;
            for (int i = threadIdx.x; i < W4; i += blockDim.x) {
                const float4 v = ld4(y + r * W, i);
                if (zero_y) st4(y + r * W, i, make_float4(0.f, 0.f, 0.f, 0.f));
                srow4[i] = v;
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
            rs_y = rsqrtf(block_sum(ss, red) / static_cast<float>(W) + eps);
        }
        float ss = 0.f;
        for (int i = threadIdx.x; i < W4; i += blockDim.x) {
            float4 v = ld4(hr, i);
            if (y) {
                const float4 a = srow4[i];
                float4 wp = ld4(w_post, i);
                if (post_scale) {
                    const float4 l4 = ld4(post_scale, i);
                    wp.x *= l4.x, wp.y *= l4.y, wp.z *= l4.z, wp.w *= l4.w;
                }
                v.x += a.x * rs_y * wp.x, v.y += a.y * rs_y * wp.y, v.z += a.z * rs_y * wp.z, v.w += a.w * rs_y * wp.w;
            }
            if (vec) {
                const float4 b = ld4(vec, i);
                v.x += b.x, v.y += b.y, v.z += b.z, v.w += b.w;
            }
            if ((y || vec) && !rows) st4(hr, i, v);
            srow4[i] = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        if (!out) return;
        OT* o = out + static_cast<long long>(t) * W;
        if (!w_pre) {
            for (int i = threadIdx.x; i < W4; i += blockDim.x) {   // each thread re-reads what it wrote itself
                const float4 a = srow4[i];
                st4(o, i, make_float4(a.x * out_scale, a.y * out_scale, a.z * out_scale, a.w * out_scale));
            }
            return;
        }
        const float rs = rsqrtf(block_sum(ss, red) / static_cast<float>(W) + eps) * out_scale;
        for (int i = threadIdx.x; i < W4; i += blockDim.x) {
            const float4 a = srow4[i], wq = ld4(w_pre, i);
            st4(o, i, make_float4(a.x * rs * wq.x, a.y * rs * wq.y, a.z * rs * wq.z, a.w * rs * wq.w));
        }
        return;
    }
    if (y) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < W; i += blockDim.x) {
            const float v = y[r * W + i];
            if (zero_y) y[r * W + i] = 0.f;
            srow[i] = v;
            ss += v * v;
        }
        rs_y = rsqrtf(block_sum(ss, red) / static_cast<float>(W) + eps);
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float v = hr[i];
        if (y) v += srow[i] * rs_y * (post_scale ? ldf(w_post, i) * ldf(post_scale, i) : ldf(w_post, i));
        if (vec) v += ldf(vec, i);
        if ((y || vec) && !rows) hr[i] = v;
        srow[i] = v;
        ss += v * v;
    }
    if (!out) return;
    OT* o = out + static_cast<long long>(t) * W;
    if (!w_pre) {
        for (int i = threadIdx.x; i < W; i += blockDim.x) stf(o, i, srow[i] * out_scale);
        return;
    }
    const float rs = rsqrtf(block_sum(ss, red) / static_cast<float>(W) + eps) * out_scale;
    for (int i = threadIdx.x; i < W; i += blockDim.x) stf(o, i, srow[i] * rs * ldf(w_pre, i));
}

// ---- act(gate) * up --------------------------------------------------------------------------------------------------
template <typename XT>
__global__ void __launch_bounds__(256) gated_act_kernel(const float* __restrict__ gu, XT* __restrict__ out, long long total,
                                                        int I) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
         e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long t = e / I;
        const int i = static_cast<int>(e - t * I);
        const float g = gu[t * 2 * I + i], u = gu[t * 2 * I + I + i];
        stf(out, e, silu_f(g) * u);
    }
}

// The clamped form: g = min(gate, limit), u = clamp(up, -limit, limit); out = g * sigmoid(alpha g) * (u + shift).
template <typename XT>
__global__ void __launch_bounds__(256) gated_act_clamped_kernel(const float* __restrict__ gu, XT* __restrict__ out,
                                                                long long total, int I, float alpha, float limit,
                                                                float shift) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
         e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long t = e / I;
        const int i = static_cast<int>(e - t * I);
        const float g = fminf(gu[t * 2 * I + i], limit);
        const float u = fminf(fmaxf(gu[t * 2 * I + I + i], -limit), limit);
        stf(out, e, g * sigmoid_f(alpha * g) * (u + shift));
    }
}

// ---- gated RMS norm of a mixer's output --------------------------------------------------------------------------
// mode 0: out = rms(y) * w * sigmoid(g) * scale      (gate after the norm)
// mode 1: u = y * silu(g); out = rms(u) * w * scale  (gate before the norm)
// mode 2: out = rms(y) * w * silu(g) * scale         (silu gate after the norm)
// The norm runs over n / groups consecutive elements; grid (T, groups). w_shared: one weight vector of n / groups
// elements for every group instead of n weights.
template <typename XT, bool VEC>
__global__ void __launch_bounds__(1024)
gated_norm_kernel(const float* __restrict__ y, long long ldy, const float* __restrict__ gate, long long ldg,
                  const XT* __restrict__ w, XT* __restrict__ out, long long ldo, int n_group, float eps, int mode,
                  float scale, int w_shared) {
    extern __shared__ __align__(16) float sgn[];   // VEC: the group's gated values between the two passes
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const long long t = blockIdx.x;
    const int c0 = blockIdx.y * n_group;
    const float* yr = y + t * ldy + c0;
    const float* gr = gate + t * ldg + c0;
    if (!w_shared) w += c0;
    if (VEC) {   // sizes and pitches multiples of 4, pointers 16-byte aligned: four elements per access, one gate pass
        const int n4 = n_group / 4;
        float4* s4 = reinterpret_cast<float4*>(sgn);
        float ss = 0.f;
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            float4 v = ld4(yr, i);
            if (mode == 1) {
                const float4 g = ld4(gr, i);
                v.x *= silu_f(g.x), v.y *= silu_f(g.y), v.z *= silu_f(g.z), v.w *= silu_f(g.w);
            }
            s4[i] = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        const float rs = rsqrtf(block_sum(ss, red) / static_cast<float>(n_group) + eps) * scale;
        XT* o = out + t * ldo + c0;
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            float4 v = s4[i];
            const float4 ww = ld4(w, i);
            v.x *= rs * ww.x, v.y *= rs * ww.y, v.z *= rs * ww.z, v.w *= rs * ww.w;
            if (mode == 0) {
                const float4 g = ld4(gr, i);
                v.x *= sigmoid_f(g.x), v.y *= sigmoid_f(g.y), v.z *= sigmoid_f(g.z), v.w *= sigmoid_f(g.w);
            } else if (mode == 2) {
                const float4 g = ld4(gr, i);
                v.x *= silu_f(g.x), v.y *= silu_f(g.y), v.z *= silu_f(g.z), v.w *= silu_f(g.w);
            }
            st4(o, i, v);
        }
        return;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < n_group; i += blockDim.x) {
        float v = yr[i];
        if (mode == 1) v *= silu_f(gr[i]);
        ss += v * v;
    }
    const float rs = rsqrtf(block_sum(ss, red) / static_cast<float>(n_group) + eps);
    XT* o = out + t * ldo + c0;
    for (int i = threadIdx.x; i < n_group; i += blockDim.x) {
        float v = yr[i];
        if (mode == 1)
            v = v * silu_f(gr[i]) * rs * ldf(w, i);
        else
            v = v * rs * ldf(w, i) * (mode == 2 ? silu_f(gr[i]) : sigmoid_f(gr[i]));
        stf(o, i, v * scale);
    }
}

// The same for narrow groups (a norm per head): a CTA per row, a warp per group and a lane per four elements, so that a row
// of many heads is one CTA instead of one small CTA per head. n_group a multiple of 4, at most 128; pointers and pitches as
// for the four-element path above.
template <typename XT>
__global__ void __launch_bounds__(256)
gated_norm_warp_kernel(const float* __restrict__ y, long long ldy, const float* __restrict__ gate, long long ldg,
                       const XT* __restrict__ w, XT* __restrict__ out, long long ldo, int n_group, int groups, float eps,
                       int mode, float scale, int w_shared) {
    pdl_launch_dependents();
    pdl_wait();
    const long long t = blockIdx.x;
    const int lane = threadIdx.x & 31, n4 = n_group / 4;
    const bool on = lane < n4;
    for (int gidx = threadIdx.x >> 5; gidx < groups; gidx += blockDim.x >> 5) {
        const int c0 = gidx * n_group;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f), g = v;
        if (on) {
            v = ld4(y + t * ldy + c0, lane);
            g = ld4(gate + t * ldg + c0, lane);
            if (mode == 1) v.x *= silu_f(g.x), v.y *= silu_f(g.y), v.z *= silu_f(g.z), v.w *= silu_f(g.w);
        }
        const float rs = rsqrtf(warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w) / static_cast<float>(n_group) + eps) * scale;
        if (!on) continue;
        const float4 ww = ld4(w_shared ? w : w + c0, lane);
        v.x *= rs * ww.x, v.y *= rs * ww.y, v.z *= rs * ww.z, v.w *= rs * ww.w;
        if (mode == 0)
            v.x *= sigmoid_f(g.x), v.y *= sigmoid_f(g.y), v.z *= sigmoid_f(g.z), v.w *= sigmoid_f(g.w);
        else if (mode == 2)
            v.x *= silu_f(g.x), v.y *= silu_f(g.y), v.z *= silu_f(g.z), v.w *= silu_f(g.w);
        st4(out + t * ldo + c0, lane, v);
    }
}

// ---- short causal convolution + silu, step size and decay of the selective scan -------------------------------------
// Channel c of row t: out = silu(b[c] + sum_j w[c][j] * in[row(t) - (K-1-j)]), the last tap being the row itself. Inputs
// before the step's first row come from the carried window conv_state[slot][K-1][C] (raw inputs of the last K-1
// positions), inputs before position 0 are zero. Columns [C, C + H) of the same launch compute, per head,
// dt = softplus(raw + dt_bias) and the decay exp(-exp(A_log) * dt).
template <typename XT>
__global__ void __launch_bounds__(256)
conv_dt_kernel(const float* __restrict__ in, long long ld, int x_off, int dt_off, const XT* __restrict__ w,
               const XT* __restrict__ b, const XT* __restrict__ dt_bias, const XT* __restrict__ a_log,
               const float* __restrict__ conv_state, float* __restrict__ xbc, float* __restrict__ dt_out,
               float* __restrict__ decay_out, const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
               const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot, int C, int H, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const long long t = blockIdx.x;
    const int s = tok_seq[t];
    if (s < 0) return;
    const int i = static_cast<int>(t) - seq_start[s];
    const int pos0 = seq_pos0[s];
    const float* st = conv_state + static_cast<long long>(seq_slot[s]) * (K - 1) * C;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C + H; c += gridDim.y * blockDim.x) {
        if (c < C) {
            float acc = ldf(b, c);
            for (int j = 0; j < K; ++j) {
                const int rel = i - (K - 1 - j);
                float v = 0.f;
                if (rel >= 0)
                    v = in[(t - i + rel) * ld + x_off + c];
                else if (pos0 + rel >= 0)
                    v = st[static_cast<long long>(K - 1 + rel) * C + c];
                acc = fmaf(ldf(w, static_cast<long long>(c) * K + j), v, acc);
            }
            xbc[t * C + c] = silu_f(acc);
        } else {
            const int hh = c - C;
            const float z = in[t * ld + dt_off + hh] + ldf(dt_bias, hh);
            const float dt = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));  // softplus, exact for every z
            dt_out[t * H + hh] = dt;
            decay_out[t * H + hh] = expf(-expf(ldf(a_log, hh)) * dt);
        }
    }
}

// The same for prompt-sized steps: a CTA takes kConvRows consecutive rows x 256 channels and every thread walks its channel
// down the rows with the taps' window in registers, so that each input and each weight is read once per tile instead
// of once per row (one CTA per row re-reads the K-1 earlier rows and all weights from L2). The window is refilled from
// the rows before the tile, or from the carried state, wherever a sequence starts or the rows are not consecutive.
constexpr int kConvRows = 16, kConvMaxTaps = 8;

// KT: the number of taps when it is one of the common ones (loops and window fold at compile time), 0: read K.
template <typename XT, int KT>
__global__ void __launch_bounds__(256)
conv_dt_tile_kernel(const float* __restrict__ in, long long ld, int x_off, int dt_off, const XT* __restrict__ w,
                    const XT* __restrict__ b, const XT* __restrict__ dt_bias, const XT* __restrict__ a_log,
                    const float* __restrict__ conv_state, float* __restrict__ xbc, float* __restrict__ dt_out,
                    float* __restrict__ decay_out, const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                    const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot, int T, int C, int H, int K_rt) {
    constexpr int MT = KT ? KT : kConvMaxTaps;   // registers for taps and window
    const int K = KT ? KT : K_rt;
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * kConvRows;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C + H) return;
    if (c >= C) {
        const int hh = c - C;
        const float bias = ldf(dt_bias, hh), rate = expf(ldf(a_log, hh));
        for (int r = 0; r < kConvRows && t0 + r < T; ++r) {
            const long long t = t0 + r;
            if (tok_seq[t] < 0) continue;
            const float z = in[t * ld + dt_off + hh] + bias;
            const float dt = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));
            dt_out[t * H + hh] = dt;
            decay_out[t * H + hh] = expf(-rate * dt);
        }
        return;
    }
    float raw[kConvRows];
#pragma unroll
    for (int r = 0; r < kConvRows; ++r) raw[r] = (t0 + r < T) ? in[static_cast<long long>(t0 + r) * ld + x_off + c] : 0.f;
    float wt[MT], win[MT > 1 ? MT - 1 : 1];
#pragma unroll
    for (int j = 0; j < MT; ++j) wt[j] = j < K ? ldf(w, static_cast<long long>(c) * K + j) : 0.f;
    const float bias = ldf(b, c);
    int prev_s = -1, prev_i = -2;
#pragma unroll
    for (int r = 0; r < kConvRows; ++r) {
        const long long t = t0 + r;
        if (t >= T) break;
        const int s = tok_seq[t];
        if (s < 0) continue;
        const int i = static_cast<int>(t) - seq_start[s];
        if (s != prev_s || i != prev_i + 1) {
            const int pos0 = seq_pos0[s];
            const float* st = conv_state + static_cast<long long>(seq_slot[s]) * (K - 1) * C;
#pragma unroll
            for (int j = 0; j < MT - 1; ++j) {
                const int rel = i - (K - 1) + j;   // row of the sequence's portion that tap j reads (negative: before it)
                float x = 0.f;
                if (j < K - 1) {
                    if (rel >= 0)
                        x = in[(t - i + rel) * ld + x_off + c];
                    else if (pos0 + rel >= 0)
                        x = st[static_cast<long long>(K - 1 + rel) * C + c];
                }
                win[j] = x;
            }
        }
        float acc = bias;
#pragma unroll
        for (int j = 0; j < MT - 1; ++j)
            if (j < K - 1) acc = fmaf(wt[j], win[j], acc);
        float wl = 0.f;
#pragma unroll
        for (int j = 0; j < MT; ++j)
            if (j == K - 1) wl = wt[j];
        acc = fmaf(wl, raw[r], acc);
        // bf16 models: the activation of a short convolution may be bf16-accurate, so the fast exponential and division
        xbc[t * C + c] = sizeof(XT) == 2 ? __fdividef(acc, 1.f + __expf(-acc)) : silu_f(acc);
        // slide: the window's entries 0 .. K-2 hold the K-1 inputs before the next row
#pragma unroll
        for (int j = 0; j < MT - 2; ++j)
            if (j < K - 2) win[j] = win[j + 1];
#pragma unroll
        for (int j = 0; j < MT - 1; ++j)
            if (j == K - 2) win[j] = raw[r];
        prev_s = s;
        prev_i = i;
    }
}

// The carried window after the step: the raw inputs of the sequence's last K-1 positions. One thread per channel walks
// the window front to back, so that a step shorter than the window shifts it in place.
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const float* __restrict__ in, long long ld, int x_off, float* __restrict__ conv_state,
                         const int* __restrict__ seq_start, const int* __restrict__ seq_count,
                         const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot, int C, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x;
    const int n = seq_count[s];
    if (n <= 0) return;
    const int pos0 = seq_pos0[s];
    const long long r0 = seq_start[s];
    float* st = conv_state + static_cast<long long>(seq_slot[s]) * (K - 1) * C;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        for (int i = 0; i < K - 1; ++i) {
            const int src = i + n;  // index into [old window | this step's rows]
            float v;
            if (src < K - 1)
                v = (pos0 - (K - 1) + src >= 0) ? st[static_cast<long long>(src) * C + c] : 0.f;
            else
                v = in[(r0 + src - (K - 1)) * ld + x_off + c];
            st[static_cast<long long>(i) * C + c] = v;
        }
    }
}


// ---- residual short convolution in front of a mixer ---------------------------------------------------------------------
// out[t, c] = x[t, c] + sum_j w[c][j] * x[row(t) - (K-1-j), c] (the last tap is the row itself; no bias, no activation):
// what a mixer reads is its input plus a causal convolution of it. x is the fp32 stream [T, ld]; rows before the step come
// from conv_state [slots, K-1, C] (atx_conv_state_update keeps it), rows before position 0 are zero. A CTA takes kConvRows
// consecutive rows x 256 channels; a thread walks its channel down the rows, so an input is fetched from memory once.
template <typename XT, int NV>   // NV = 4: four channels per thread with 16-byte accesses (sizes, pitches and pointers allow it)
__global__ void __launch_bounds__(256)
conv_residual_kernel(const float* __restrict__ x, long long ld, const XT* __restrict__ w, const float* __restrict__ conv_state,
                     XT* __restrict__ out, long long ldo, const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                     const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot, int T, int C, int K, int rows_per) {
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * rows_per;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * NV;
    if (c >= C) return;
    float wt[kConvMaxTaps][NV], win[kConvMaxTaps - 1][NV];
#pragma unroll
    for (int j = 0; j < kConvMaxTaps; ++j)
#pragma unroll
        for (int e = 0; e < NV; ++e) wt[j][e] = j < K ? ldf(w, static_cast<long long>(c + e) * K + j) : 0.f;
    auto load = [&](const float* p, float (&v)[NV]) {
        if (NV == 4) {
            const float4 f = *reinterpret_cast<const float4*>(p);
            v[0] = f.x, v[NV > 1 ? 1 : 0] = f.y, v[NV > 2 ? 2 : 0] = f.z, v[NV > 3 ? 3 : 0] = f.w;
        } else {
            v[0] = *p;
        }
    };
    int prev_s = -1, prev_i = -2;
    for (int r = 0; r < rows_per && t0 + r < T; ++r) {
        const long long t = t0 + r;
        const int s = tok_seq[t];
        if (s < 0) continue;
        const int i = static_cast<int>(t) - seq_start[s];
        if (s != prev_s || i != prev_i + 1) {   // the window of the K-1 rows before this one: earlier rows of the portion, or the slot
            const int pos0 = seq_pos0[s];
            const float* st = conv_state + static_cast<long long>(seq_slot[s]) * (K - 1) * C;
#pragma unroll
            for (int j = 0; j < kConvMaxTaps - 1; ++j) {
#pragma unroll
                for (int e = 0; e < NV; ++e) win[j][e] = 0.f;
                if (j < K - 1) {
                    const int rel = i - (K - 1) + j;
                    if (rel >= 0)
                        load(x + (t - i + rel) * ld + c, win[j]);
                    else if (pos0 + rel >= 0)
                        load(st + static_cast<long long>(K - 1 + rel) * C + c, win[j]);
                }
            }
        }
        float cur[NV], acc[NV];
        load(x + t * ld + c, cur);
#pragma unroll
        for (int e = 0; e < NV; ++e) acc[e] = cur[e];
#pragma unroll
        for (int j = 0; j < kConvMaxTaps - 1; ++j)
            if (j < K - 1)
#pragma unroll
                for (int e = 0; e < NV; ++e) acc[e] = fmaf(wt[j][e], win[j][e], acc[e]);
#pragma unroll
        for (int j = 0; j < kConvMaxTaps; ++j)
            if (j == K - 1)
#pragma unroll
                for (int e = 0; e < NV; ++e) acc[e] = fmaf(wt[j][e], cur[e], acc[e]);
        if (NV == 4) {
            st4(out + t * ldo + c, 0, make_float4(acc[0], acc[NV > 1 ? 1 : 0], acc[NV > 2 ? 2 : 0], acc[NV > 3 ? 3 : 0]));
        } else {
            stf(out + t * ldo, c, acc[0]);
        }
        // slide: entries 0 .. K-2 hold the K-1 inputs before the next row
#pragma unroll
        for (int j = 0; j < kConvMaxTaps - 2; ++j)
            if (j < K - 2)
#pragma unroll
                for (int e = 0; e < NV; ++e) win[j][e] = win[j + 1][e];
#pragma unroll
        for (int j = 0; j < kConvMaxTaps - 1; ++j)
            if (j == K - 2)
#pragma unroll
                for (int e = 0; e < NV; ++e) win[j][e] = cur[e];
        prev_s = s;
        prev_i = i;
    }
}

// More taps than the register window holds: a thread per (row, channel) sums its taps straight from memory.
template <typename XT>
__global__ void __launch_bounds__(256)
conv_residual_long_kernel(const float* __restrict__ x, long long ld, const XT* __restrict__ w,
                          const float* __restrict__ conv_state, XT* __restrict__ out, long long ldo,
                          const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                          const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot, int C, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const long long t = blockIdx.x;
    const int s = tok_seq[t];
    if (s < 0) return;
    const int i = static_cast<int>(t) - seq_start[s], pos0 = seq_pos0[s];
    const float* st = conv_state + static_cast<long long>(seq_slot[s]) * (K - 1) * C;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float acc = x[t * ld + c];
        for (int j = 0; j < K; ++j) {
            const int rel = i - (K - 1 - j);
            float v = 0.f;
            if (rel >= 0)
                v = x[(t - i + rel) * ld + c];
            else if (pos0 + rel >= 0)
                v = st[static_cast<long long>(K - 1 + rel) * C + c];
            acc = fmaf(ldf(w, static_cast<long long>(c) * K + j), v, acc);
        }
        stf(out + t * ldo, c, acc);
    }
}

// ---- data-dependent decay per channel through a low-rank projection -------------------------------------------------
// z[t, c] = b[c] + sum_r A[c, r] * lo[t, r];  out[t, c] = log(sigmoid(z)^(1/tau)) = -softplus(-z) / tau  (fp32, <= 0).
// lo: the fp32 output of the first (narrow) projection, R columns at pitch ld. One CTA per row tile of 8 rows; the narrow
// rows sit in shared memory and a thread owns a channel, walking its R weights once for the tile's eight rows.
template <typename XT>
__global__ void __launch_bounds__(256)
lowrank_logdecay_kernel(const float* __restrict__ lo, long long ld, const XT* __restrict__ A, const XT* __restrict__ b,
                        float* __restrict__ out, long long ldo, int T, int C, int R, float inv_tau) {
    extern __shared__ __align__(16) float slo[];   // [8][R]
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * 8;
    const int rows = min(8, T - t0);
    for (int e = threadIdx.x; e < rows * R; e += blockDim.x) {
        const int i = e / R, r = e - i * R;
        slo[e] = lo[static_cast<long long>(t0 + i) * ld + r];
    }
    __syncthreads();
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float acc[8];
        const float bias = b ? ldf(b, c) : 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = bias;
        for (int r = 0; r < R; ++r) {
            const float a = ldf(A, static_cast<long long>(c) * R + r);
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (i < rows) acc[i] = fmaf(a, slo[i * R + r], acc[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (i >= rows) break;
            const float z = acc[i];
            // log sigmoid(z) = -softplus(-z) = min(z, 0) - log1p(exp(-|z|)), exact for every z
            out[static_cast<long long>(t0 + i) * ldo + c] = (fminf(z, 0.f) - log1pf(expf(-fabsf(z)))) * inv_tau;
        }
    }
}

// packed fp32 pairs (sm_100 FFMA2 / FMUL2): two state rows per instruction
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pk2(float lo, float hi) {
    f32x2 v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
    return v;
}
__device__ __forceinline__ void upk2(f32x2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// ---- decayed outer-product recurrence ----------------------------------------------------------------------------
// Per head: S_t = a_t S_(t-1) + (c_t k_t) v_t^T (S is D x V), y_t = S_t^T q_t + d v_t.
//   a_t = decay_head[h] or decay_tok[t, h];  c_t = kscale_tok[t, h] or 1;  d = skip[h] or 0;
//   q and k of head h are read from group h / (H / G) (G = H: a q/k per head), v from head h;
//   act = 1 applies silu to q, k and v as they are read.
//   CH: the decay acts per key channel instead, a_t[d] = exp(ldecay_chan[t, h D + d]) (logarithms given, pitch ldc), and q
//   is multiplied by qscale as it is read.
// One CTA owns a V-tile of one head of one sequence and walks the sequence's rows in order. A thread keeps DS rows of
// one column of S in registers for the whole walk (the state is read once and written once per step); rows are staged
// through shared memory kChunk at a time, and the partial dot products of the D-slices are summed per chunk.
constexpr int kRecChunk = 16;

template <int DS, bool FULL, bool CH = false>   // FULL: D is a multiple of DS (no partial slice) and rows of q / k are 16-byte aligned
__global__ void __launch_bounds__(256, DS == 32 ? 2 : 1)
linear_recurrence_kernel(const float* __restrict__ q, long long ldq, const float* __restrict__ k, long long ldk,
                         const float* __restrict__ v, long long ldv, int H, int G, int D, int V,
                         const float* __restrict__ decay_head, const float* __restrict__ decay_tok,
                         const float* __restrict__ kscale_tok, const float* __restrict__ skip, int act,
                         float* __restrict__ state, float* __restrict__ y, long long ldy,
                         const int* __restrict__ seq_start, const int* __restrict__ seq_count,
                         const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot, int VT, int DG,
                         const float* __restrict__ ldecay_chan = nullptr, long long ldc = 0, float qscale = 1.f) {
    extern __shared__ __align__(16) float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y;
    const int n = seq_count[s];
    if (n <= 0) return;
    const long long r0 = seq_start[s];
    const int g = h / (H / G);
    const int tv = threadIdx.x % VT, dg = threadIdx.x / VT;
    const int col = blockIdx.z * VT + tv;
    const bool live = col < V && dg < DG;
    const int d0 = dg * DS;
    float* sq = sm;                            // [kRecChunk][D]
    float* sk = sq + kRecChunk * D;            // [kRecChunk][D]   (already scaled by c_t)
    float* sv = sk + kRecChunk * D;            // [kRecChunk][VT]
    float* sa = sv + kRecChunk * VT;           // [kRecChunk]
    float* sp = sa + kRecChunk;                // [kRecChunk][DG][VT] partial outputs
    float* sd = sp + kRecChunk * DG * VT;      // CH: [kRecChunk][D] decay factors per key channel
    float S[DS];
    float* st = state + ((static_cast<long long>(seq_slot[s]) * H + h) * D) * V;
    const bool fresh = seq_pos0[s] == 0;
#pragma unroll
    for (int i = 0; i < DS; ++i) S[i] = (live && !fresh && d0 + i < D) ? st[static_cast<long long>(d0 + i) * V + col] : 0.f;
    const float dskip = skip ? skip[h] : 0.f;
    for (int c0 = 0; c0 < n; c0 += kRecChunk) {
        const int cn = min(kRecChunk, n - c0);
        __syncthreads();
        for (int e = threadIdx.x; e < cn * D; e += blockDim.x) {
            const int i = e / D, d = e - i * D;
            const long long row = r0 + c0 + i;
            float qv = q[row * ldq + g * D + d], kv = k[row * ldk + g * D + d];
            if (act) {
                qv = silu_f(qv);
                kv = silu_f(kv);
            }
            if (kscale_tok) kv *= kscale_tok[row * H + h];
            if (CH) {
                qv *= qscale;
                sd[i * D + d] = expf(ldecay_chan[row * ldc + static_cast<long long>(h) * D + d]);
            }
            sq[i * D + d] = qv;
            sk[i * D + d] = kv;
        }
        for (int e = threadIdx.x; e < cn * VT; e += blockDim.x) {
            const int i = e / VT, j = e - i * VT;
            const int cc = blockIdx.z * VT + j;
            float vv = cc < V ? v[(r0 + c0 + i) * ldv + h * V + cc] : 0.f;
            if (act) vv = silu_f(vv);
            sv[i * VT + j] = vv;
        }
        if (!CH)
            for (int i = threadIdx.x; i < cn; i += blockDim.x)
                sa[i] = decay_tok ? decay_tok[(r0 + c0 + i) * H + h] : decay_head[h];
        __syncthreads();
        if (live) {
            for (int i = 0; i < cn; ++i) {
                const float a = CH ? 1.f : sa[i], vv = sv[i * VT + tv];
                const float* qi = sq + i * D + d0;
                const float* ki = sk + i * D + d0;
                const float* di = sd + i * D + d0;
                float acc = 0.f;
                if (FULL) {
                    // state rows in pairs: S2 = a2 * S2 + k2 * v2; acc2 += S2 * q2  (three packed operations per pair),
                    // four independent accumulators so that the dot product is not one dependent chain
                    const ulonglong2* q4 = reinterpret_cast<const ulonglong2*>(qi);
                    const ulonglong2* k4 = reinterpret_cast<const ulonglong2*>(ki);
                    const ulonglong2* d4 = reinterpret_cast<const ulonglong2*>(di);
                    const f32x2 a2 = pk2(a, a), v2 = pk2(vv, vv);
                    f32x2 ac[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
                    for (int d = 0; d < DS / 4; ++d) {
                        const ulonglong2 kk = k4[d], qq = q4[d];
                        f32x2 s0 = pk2(S[4 * d], S[4 * d + 1]), s1 = pk2(S[4 * d + 2], S[4 * d + 3]);
                        if (CH) {
                            const ulonglong2 dd = d4[d];
                            s0 = fma2(dd.x, s0, mul2(kk.x, v2));
                            s1 = fma2(dd.y, s1, mul2(kk.y, v2));
                        } else {
                            s0 = fma2(a2, s0, mul2(kk.x, v2));
                            s1 = fma2(a2, s1, mul2(kk.y, v2));
                        }
                        ac[(2 * d) & 3] = fma2(s0, qq.x, ac[(2 * d) & 3]);
                        ac[(2 * d + 1) & 3] = fma2(s1, qq.y, ac[(2 * d + 1) & 3]);
                        upk2(s0, S[4 * d], S[4 * d + 1]);
                        upk2(s1, S[4 * d + 2], S[4 * d + 3]);
                    }
                    float x0, x1, x2, x3, x4, x5, x6, x7;
                    upk2(ac[0], x0, x1);
                    upk2(ac[1], x2, x3);
                    upk2(ac[2], x4, x5);
                    upk2(ac[3], x6, x7);
                    acc = ((x0 + x1) + (x2 + x3)) + ((x4 + x5) + (x6 + x7));
                } else {
#pragma unroll
                    for (int d = 0; d < DS; ++d) {
                        if (d0 + d < D) {
                            S[d] = fmaf(CH ? di[d] : a, S[d], ki[d] * vv);
                            acc = fmaf(S[d], qi[d], acc);
                        }
                    }
                }
                sp[(i * DG + dg) * VT + tv] = acc;
            }
        }
        __syncthreads();
        for (int e = threadIdx.x; e < cn * VT; e += blockDim.x) {
            const int i = e / VT, j = e - i * VT;
            const int cc = blockIdx.z * VT + j;
            if (cc >= V) continue;
            float acc = dskip * sv[i * VT + j];
            for (int z = 0; z < DG; ++z) acc += sp[(i * DG + z) * VT + j];
            y[(r0 + c0 + i) * ldy + h * V + cc] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < DS; ++i)
            if (d0 + i < D) st[static_cast<long long>(d0 + i) * V + col] = S[i];
    }
}

}  // namespace atx

using namespace atx;

#define ATX_DISPATCH_XT(dtype, ...)                                  \
    do {                                                             \
        if ((dtype) == ATX_DT_F32) {                                 \
            using XT = float;                                        \
            __VA_ARGS__;                                             \
        } else {                                                     \
            using XT = __nv_bfloat16;                                \
            __VA_ARGS__;                                             \
        }                                                            \
    } while (0)

extern "C" {

int atx_embed_rows(const int* ids, const void* table, float* out, int T, int W, int V, int dtype, int flags,
                   atx_stream_t stream) {
    return atx_embed_rows_scaled(ids, table, out, T, W, V, 1.f, dtype, flags, stream);
}

int atx_embed_rows_scaled(const int* ids, const void* table, float* out, int T, int W, int V, float scale, int dtype,
                          int flags, atx_stream_t stream) {
    ATX_REQUIRE(ids && table && out, "atx_embed_rows: null pointer");
    ATX_REQUIRE(T > 0 && W > 0 && V > 0, "atx_embed_rows: bad shape T=%d W=%d V=%d", T, W, V);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(T);
    cfg.blockDim = dim3(128);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl2(cfg, attr, flags);
    ATX_DISPATCH_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(&cfg, embed_rows_kernel<XT>, ids,
                                                       reinterpret_cast<const XT*>(table), out, W, V, scale)));
    return ATX_OK;
}

int atx_concat_embed(const float* h, const int* ids, const void* table, void* out, int T, int W, int V, int dtype,
                     int flags, atx_stream_t stream) {
    ATX_REQUIRE(h && ids && table && out, "atx_concat_embed: null pointer");
    ATX_REQUIRE(T > 0 && W > 0 && V > 0, "atx_concat_embed: bad shape T=%d W=%d V=%d", T, W, V);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(T);
    cfg.blockDim = dim3(128);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl2(cfg, attr, flags);
    ATX_DISPATCH_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(&cfg, concat_embed_kernel<XT>, h, ids,
                                                       reinterpret_cast<const XT*>(table), reinterpret_cast<XT*>(out),
                                                       W, V)));
    return ATX_OK;
}

int atx_resid_norm(float* h, float* y, const void* w_post, const void* vec, const void* w_pre, void* out,
                   const int* rows, int T, int W, float eps, int zero_y, void* zero_ptr, long long zero_bytes, int dtype,
                   int flags, atx_stream_t stream) {
    return atx_resid_norm_scaled(h, y, w_post, nullptr, vec, w_pre, out, 0, rows, T, W, eps, zero_y, zero_ptr, zero_bytes,
                                 dtype, flags, stream);
}

int atx_resid_norm_scaled(float* h, float* y, const void* w_post, const void* post_scale, const void* vec,
                          const void* w_pre, void* out, int out_f32, const int* rows, int T, int W, float eps, int zero_y,
                          void* zero_ptr, long long zero_bytes, int dtype, int flags, atx_stream_t stream) {
    ATX_REQUIRE((w_pre == nullptr) == (out == nullptr), "atx_resid_norm: w_pre and out come together");
    return atx_resid_norm_out(h, y, w_post, post_scale, vec, w_pre, out, out_f32, 1.f, rows, T, W, eps, zero_y, zero_ptr,
                              zero_bytes, dtype, flags, stream);
}

int atx_resid_norm_out(float* h, float* y, const void* w_post, const void* post_scale, const void* vec, const void* w_pre,
                       void* out, int out_f32, float out_scale, const int* rows, int T, int W, float eps, int zero_y,
                       void* zero_ptr, long long zero_bytes, int dtype, int flags, atx_stream_t stream) {
    ATX_REQUIRE(h, "atx_resid_norm: null pointer");
    ATX_REQUIRE(!post_scale || w_post, "atx_resid_norm: post_scale needs y and w_post");
    ATX_REQUIRE(T > 0 && W > 0 && W <= 12288, "atx_resid_norm: bad shape T=%d W=%d (W <= 12288)", T, W);
    ATX_REQUIRE((y == nullptr) == (w_post == nullptr), "atx_resid_norm: y and w_post come together");
    ATX_REQUIRE(!w_pre || out, "atx_resid_norm: w_pre needs out");
    ATX_REQUIRE(zero_bytes >= 0 && zero_bytes % 16 == 0 && (zero_bytes == 0 || zero_ptr) && !(zero_y && rows),
                "atx_resid_norm: zero_bytes=%lld must be a non-negative multiple of 16 with a buffer; zero_y not with rows",
                zero_bytes);
    const long long zv = zero_bytes / 16;
    long long zb = (zv + 256 * 8 - 1) / (256 * 8);
    if (zb > 2048) zb = 2048;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(static_cast<unsigned>(T + zb));
    cfg.blockDim = dim3(T <= 512 && W >= 2048 ? 1024 : 256);   // few rows: more warps per row hide the load latency
    cfg.dynamicSmemBytes = static_cast<size_t>(W) * 4;
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl2(cfg, attr, flags);
    auto al16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const bool v4 = W % 4 == 0 && al16(h) && al16(y) && al16(w_post) && al16(post_scale) && al16(vec) && al16(w_pre) &&
                    al16(out);
#define ATX_RESID(OT_, VEC_)                                                                                              \
    ATX_DISPATCH_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(                                                                   \
                               &cfg, resid_norm_kernel<XT, OT_, VEC_>, h, y, reinterpret_cast<const XT*>(w_post),         \
                               reinterpret_cast<const XT*>(post_scale), reinterpret_cast<const XT*>(vec),                 \
                               reinterpret_cast<const XT*>(w_pre), reinterpret_cast<OT_*>(out), rows, T, W, eps, zero_y,  \
                               reinterpret_cast<uint4*>(zero_ptr), zv, out_scale)))
    if (out_f32) {
        if (v4)
            ATX_RESID(float, true);
        else
            ATX_RESID(float, false);
    } else {
        if (v4)
            ATX_RESID(XT, true);
        else
            ATX_RESID(XT, false);
    }
#undef ATX_RESID
    return ATX_OK;
}

int atx_gated_act(const float* gu, void* out, int T, int I, int dtype, int flags, atx_stream_t stream) {
    ATX_REQUIRE(gu && out, "atx_gated_act: null pointer");
    ATX_REQUIRE(T > 0 && I > 0, "atx_gated_act: bad shape T=%d I=%d", T, I);
    const long long total = static_cast<long long>(T) * I;
    long long blocks = (total + 255) / 256;
    const long long cap = static_cast<long long>(num_sms()) * 16;
    if (blocks > cap) blocks = cap;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(static_cast<unsigned>(blocks));
    cfg.blockDim = dim3(256);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl2(cfg, attr, flags);
    ATX_DISPATCH_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(&cfg, gated_act_kernel<XT>, gu, reinterpret_cast<XT*>(out), total, I)));
    return ATX_OK;
}

int atx_gated_act_clamped(const float* gu, void* out, int T, int I, float alpha, float limit, float shift, int dtype,
                          int flags, atx_stream_t stream) {
    ATX_REQUIRE(gu && out, "atx_gated_act_clamped: null pointer");
    ATX_REQUIRE(T > 0 && I > 0 && limit > 0.f, "atx_gated_act_clamped: bad arguments T=%d I=%d limit=%g", T, I, limit);
    const long long total = static_cast<long long>(T) * I;
    long long blocks = (total + 255) / 256;
    const long long cap = static_cast<long long>(num_sms()) * 16;
    if (blocks > cap) blocks = cap;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(static_cast<unsigned>(blocks));
    cfg.blockDim = dim3(256);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl2(cfg, attr, flags);
    ATX_DISPATCH_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(&cfg, gated_act_clamped_kernel<XT>, gu, reinterpret_cast<XT*>(out),
                                                       total, I, alpha, limit, shift)));
    return ATX_OK;
}

int atx_gated_norm(const float* y, long long ldy, const float* gate, long long ldg, const void* w, void* out,
                   long long ldo, int T, int n, int groups, float eps, int mode, float scale, int dtype, int flags,
                   atx_stream_t stream) {
    return atx_gated_norm_groups(y, ldy, gate, ldg, w, 0, out, ldo, T, n, groups, eps, mode, scale, dtype, flags, stream);
}

int atx_gated_norm_groups(const float* y, long long ldy, const float* gate, long long ldg, const void* w, int w_shared,
                          void* out, long long ldo, int T, int n, int groups, float eps, int mode, float scale, int dtype,
                          int flags, atx_stream_t stream) {
    ATX_REQUIRE(y && gate && w && out, "atx_gated_norm: null pointer");
    ATX_REQUIRE(T > 0 && n > 0 && groups > 0 && n % groups == 0 && mode >= 0 && mode <= 2,
                "atx_gated_norm: bad arguments T=%d n=%d groups=%d mode=%d", T, n, groups, mode);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(T, groups);
    // a thread takes four elements at a time: narrow groups (a norm per head) get a CTA of as many warps as that needs
    const int lanes = (n / groups + 3) / 4;
    cfg.blockDim = dim3(T <= 512 && n / groups >= 2048 ? 1024 : lanes <= 32 ? 32 : lanes <= 64 ? 64 : lanes <= 128 ? 128 : 256);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl2(cfg, attr, flags);
    auto al16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const int ng = n / groups;
    const bool v4 = ng % 4 == 0 && ldy % 4 == 0 && ldg % 4 == 0 && ldo % 4 == 0 && al16(y) && al16(gate) && al16(w) &&
                    al16(out) && ng * 4 <= 96 * 1024;
#define ATX_GNORM(VEC_)                                                                                                  \
    ATX_DISPATCH_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(&cfg, gated_norm_kernel<XT, VEC_>, y, ldy, gate, ldg,             \
                                                       reinterpret_cast<const XT*>(w), reinterpret_cast<XT*>(out), ldo,  \
                                                       ng, eps, mode, scale, w_shared)))
    if (v4 && ng <= 128 && groups > 1) {
        cfg.gridDim = dim3(T);
        cfg.blockDim = dim3(groups >= 8 ? 256 : 32 * groups);
        ATX_DISPATCH_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(&cfg, gated_norm_warp_kernel<XT>, y, ldy, gate, ldg,
                                                           reinterpret_cast<const XT*>(w), reinterpret_cast<XT*>(out), ldo,
                                                           ng, groups, eps, mode, scale, w_shared)));
        return ATX_OK;
    }
    if (v4) {
        cfg.dynamicSmemBytes = static_cast<size_t>(ng) * 4;
        if (ng * 4 > 48 * 1024) {
            ATX_DISPATCH_XT(dtype, ATX_CUDA(cudaFuncSetAttribute(gated_norm_kernel<XT, true>,
                                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024)));
        }
        ATX_GNORM(true);
    } else {
        ATX_GNORM(false);
    }
#undef ATX_GNORM
    return ATX_OK;
}

int atx_conv_dt(const float* in, long long ld, int x_off, int dt_off, const void* w, const void* b, const void* dt_bias,
                const void* a_log, const float* conv_state, float* xbc, float* dt_out, float* decay_out,
                const int* tok_seq, const int* seq_start, const int* seq_pos0, const int* seq_slot, int T, int C, int H,
                int K, int dtype, int flags, atx_stream_t stream) {
    ATX_REQUIRE(in && w && b && dt_bias && a_log && conv_state && xbc && dt_out && decay_out && tok_seq && seq_start &&
                    seq_pos0 && seq_slot,
                "atx_conv_dt: null pointer");
    ATX_REQUIRE(T > 0 && C > 0 && H > 0 && K >= 1, "atx_conv_dt: bad shape T=%d C=%d H=%d K=%d", T, C, H, K);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    // few rows (decode): spread a row's channels over several CTAs
    cfg.gridDim = dim3(T, T >= 256 ? 1 : (C + H + 255) / 256);
    cfg.blockDim = dim3(256);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl2(cfg, attr, flags);
    if (T >= 256 && K >= 2 && K <= kConvMaxTaps) {
        cfg.gridDim = dim3((T + kConvRows - 1) / kConvRows, (C + H + 255) / 256);
#define ATX_CONV_TILE(KT_)                                                                                                \
    ATX_DISPATCH_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(                                                                   \
                               &cfg, conv_dt_tile_kernel<XT, KT_>, in, ld, x_off, dt_off, reinterpret_cast<const XT*>(w), \
                               reinterpret_cast<const XT*>(b), reinterpret_cast<const XT*>(dt_bias),                      \
                               reinterpret_cast<const XT*>(a_log), conv_state, xbc, dt_out, decay_out, tok_seq,           \
                               seq_start, seq_pos0, seq_slot, T, C, H, K)))
        if (K == 4)
            ATX_CONV_TILE(4);
        else if (K == 3)
            ATX_CONV_TILE(3);
        else if (K == 2)
            ATX_CONV_TILE(2);
        else
            ATX_CONV_TILE(0);
#undef ATX_CONV_TILE
        return ATX_OK;
    }
    ATX_DISPATCH_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(
                               &cfg, conv_dt_kernel<XT>, in, ld, x_off, dt_off, reinterpret_cast<const XT*>(w),
                               reinterpret_cast<const XT*>(b), reinterpret_cast<const XT*>(dt_bias),
                               reinterpret_cast<const XT*>(a_log), conv_state, xbc, dt_out, decay_out, tok_seq,
                               seq_start, seq_pos0, seq_slot, C, H, K)));
    return ATX_OK;
}

int atx_conv_state_update(const float* in, long long ld, int x_off, float* conv_state, const int* seq_start,
                          const int* seq_count, const int* seq_pos0, const int* seq_slot, int n_seqs, int C, int K,
                          int flags, atx_stream_t stream) {
    ATX_REQUIRE(in && conv_state && seq_start && seq_count && seq_pos0 && seq_slot, "atx_conv_state_update: null pointer");
    ATX_REQUIRE(n_seqs > 0 && C > 0 && K >= 1, "atx_conv_state_update: bad shape n_seqs=%d C=%d K=%d", n_seqs, C, K);
    if (K == 1) return ATX_OK;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(n_seqs, (C + 255) / 256);
    cfg.blockDim = dim3(256);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl2(cfg, attr, flags);
    ATX_CUDA(cudaLaunchKernelEx(&cfg, conv_state_update_kernel, in, ld, x_off, conv_state, seq_start, seq_count, seq_pos0,
                                seq_slot, C, K));
    return ATX_OK;
}

int atx_linear_recurrence(const float* q, long long ldq, const float* k, long long ldk, const float* v, long long ldv,
                          int H, int G, int D, int V, const float* decay_head, const float* decay_tok,
                          const float* kscale_tok, const float* skip, int act, float* state, float* y, long long ldy,
                          const int* seq_start, const int* seq_count, const int* seq_pos0, const int* seq_slot,
                          int n_seqs, int flags, atx_stream_t stream) {
    ATX_REQUIRE(q && k && v && state && y && seq_start && seq_count && seq_pos0 && seq_slot,
                "atx_linear_recurrence: null pointer");
    ATX_REQUIRE((decay_head != nullptr) != (decay_tok != nullptr),
                "atx_linear_recurrence: exactly one of decay_head / decay_tok");
    ATX_REQUIRE(n_seqs > 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && V > 0 && D <= 512,
                "atx_linear_recurrence: bad shape n_seqs=%d H=%d G=%d D=%d V=%d (D <= 512)", n_seqs, H, G, D, V);
    const int DS = D > 256 ? 64 : 32;
    const int DG = (D + DS - 1) / DS;
    int VT = (256 / DG) / 32 * 32;
    if (VT < 32) VT = 32;
    const int v32 = (V + 31) / 32 * 32;
    if (VT > v32) VT = v32;
    const int threads = VT * DG;
    const size_t smem = sizeof(float) * (static_cast<size_t>(kRecChunk) * (2 * D + VT + 1 + DG * VT));
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(n_seqs, H, (V + VT - 1) / VT);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl2(cfg, attr, flags);
    ATX_REQUIRE(smem <= 160 * 1024, "atx_linear_recurrence: D=%d needs %zu bytes of shared memory", D, smem);
    const bool full = D % DS == 0 && D % 4 == 0;
#define ATX_REC_LAUNCH(DS_, FULL_)                                                                                       \
    do {                                                                                                                  \
        if (smem > 48 * 1024)                                                                                             \
            ATX_CUDA(cudaFuncSetAttribute(linear_recurrence_kernel<DS_, FULL_>,                                           \
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));          \
        ATX_CUDA(cudaLaunchKernelEx(&cfg, linear_recurrence_kernel<DS_, FULL_>, q, ldq, k, ldk, v, ldv, H, G, D, V,       \
                                    decay_head, decay_tok, kscale_tok, skip, act, state, y, ldy, seq_start, seq_count,   \
                                    seq_pos0, seq_slot, VT, DG, static_cast<const float*>(nullptr), 0LL, 1.f)); \
    } while (0)
    if (DS == 32 && full)
        ATX_REC_LAUNCH(32, true);
    else if (DS == 32)
        ATX_REC_LAUNCH(32, false);
    else if (full)
        ATX_REC_LAUNCH(64, true);
    else
        ATX_REC_LAUNCH(64, false);
#undef ATX_REC_LAUNCH
    return ATX_OK;
}

int atx_conv_residual(const float* x, long long ld, const void* w, const float* conv_state, void* out, long long ldo,
                      const int* tok_seq, const int* seq_start, const int* seq_pos0, const int* seq_slot, int T, int C,
                      int K, int dtype, int flags, atx_stream_t stream) {
    ATX_REQUIRE(x && w && out && tok_seq && seq_start && seq_pos0 && seq_slot && (K == 1 || conv_state),
                "atx_conv_residual: null pointer");
    ATX_REQUIRE(T > 0 && C > 0 && K >= 1, "atx_conv_residual: bad shape T=%d C=%d taps=%d", T, C, K);
    if (K > kConvMaxTaps) {
        cudaLaunchConfig_t lc = {};
        cudaLaunchAttribute la[1];
        lc.gridDim = dim3(T, (C + 255) / 256);
        lc.blockDim = dim3(256);
        lc.stream = reinterpret_cast<cudaStream_t>(stream);
        set_pdl2(lc, la, flags);
        ATX_DISPATCH_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(&lc, conv_residual_long_kernel<XT>, x, ld,
                                                           reinterpret_cast<const XT*>(w), conv_state,
                                                           reinterpret_cast<XT*>(out), ldo, tok_seq, seq_start, seq_pos0,
                                                           seq_slot, C, K)));
        return ATX_OK;
    }
    const int rows_per = T >= 256 ? kConvRows : 1;   // few rows (decode): a CTA per row
    auto al16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const bool v4 = C % 4 == 0 && ld % 4 == 0 && ldo % 4 == 0 && al16(x) && al16(out) && (K == 1 || al16(conv_state));
    const int per_cta = v4 ? 128 * 4 : 256;          // channels a CTA covers
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3((T + rows_per - 1) / rows_per, (C + per_cta - 1) / per_cta);
    cfg.blockDim = dim3(v4 ? 128 : 256);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl2(cfg, attr, flags);
#define ATX_CONV_RES(NV_)                                                                                                  \
    ATX_DISPATCH_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(&cfg, conv_residual_kernel<XT, NV_>, x, ld,                         \
                                                       reinterpret_cast<const XT*>(w), conv_state,                         \
                                                       reinterpret_cast<XT*>(out), ldo, tok_seq, seq_start, seq_pos0,      \
                                                       seq_slot, T, C, K, rows_per)))
    if (v4)
        ATX_CONV_RES(4);
    else
        ATX_CONV_RES(1);
#undef ATX_CONV_RES
    return ATX_OK;
}

int atx_lowrank_logdecay(const float* lo, long long ld, const void* A, const void* b, float* out, long long ldo, int T,
                         int C, int R, float tau, int dtype, int flags, atx_stream_t stream) {
    ATX_REQUIRE(lo && A && out, "atx_lowrank_logdecay: null pointer");
    ATX_REQUIRE(T > 0 && C > 0 && R > 0 && R <= 4096 && tau > 0.f, "atx_lowrank_logdecay: bad arguments T=%d C=%d R=%d tau=%g",
                T, C, R, tau);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3((T + 7) / 8, (C + 255) / 256);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = sizeof(float) * 8 * static_cast<size_t>(R);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl2(cfg, attr, flags);
    const float inv_tau = 1.f / tau;
    ATX_DISPATCH_XT(dtype, ATX_CUDA(cudaLaunchKernelEx(&cfg, lowrank_logdecay_kernel<XT>, lo, ld,
                                                       reinterpret_cast<const XT*>(A), reinterpret_cast<const XT*>(b), out,
                                                       ldo, T, C, R, inv_tau)));
    return ATX_OK;
}

int atx_gated_linear_recurrence(const float* q, long long ldq, const float* k, long long ldk, const float* v, long long ldv,
                                const float* ldecay, long long ldc, int H, int D, int V, float qscale, float* state,
                                float* y, long long ldy, const int* seq_start, const int* seq_count, const int* seq_pos0,
                                const int* seq_slot, int n_seqs, int flags, atx_stream_t stream) {
    ATX_REQUIRE(q && k && v && ldecay && state && y && seq_start && seq_count && seq_pos0 && seq_slot,
                "atx_gated_linear_recurrence: null pointer");
    ATX_REQUIRE(n_seqs > 0 && H > 0 && D > 0 && V > 0 && D <= 512,
                "atx_gated_linear_recurrence: bad shape n_seqs=%d H=%d D=%d V=%d (D <= 512)", n_seqs, H, D, V);
    const int DS = D > 256 ? 64 : 32;
    const int DG = (D + DS - 1) / DS;
    int VT = (256 / DG) / 32 * 32;
    if (VT < 32) VT = 32;
    const int v32 = (V + 31) / 32 * 32;
    if (VT > v32) VT = v32;
    const int threads = VT * DG;
    const size_t smem = sizeof(float) * (static_cast<size_t>(kRecChunk) * (3 * D + VT + 1 + DG * VT));
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(n_seqs, H, (V + VT - 1) / VT);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl2(cfg, attr, flags);
    ATX_REQUIRE(smem <= 160 * 1024, "atx_gated_linear_recurrence: D=%d needs %zu bytes of shared memory", D, smem);
    const bool full = D % DS == 0 && D % 4 == 0;
    const float* none = nullptr;
#define ATX_GREC_LAUNCH(DS_, FULL_)                                                                                      \
    do {                                                                                                                  \
        if (smem > 48 * 1024)                                                                                             \
            ATX_CUDA(cudaFuncSetAttribute(linear_recurrence_kernel<DS_, FULL_, true>,                                     \
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));          \
        ATX_CUDA(cudaLaunchKernelEx(&cfg, linear_recurrence_kernel<DS_, FULL_, true>, q, ldq, k, ldk, v, ldv, H, H, D, V, \
                                    none, none, none, none, 0, state, y, ldy, seq_start, seq_count, seq_pos0, seq_slot,  \
                                    VT, DG, ldecay, ldc, qscale));                                                        \
    } while (0)
    if (DS == 32 && full)
        ATX_GREC_LAUNCH(32, true);
    else if (DS == 32)
        ATX_GREC_LAUNCH(32, false);
    else if (full)
        ATX_GREC_LAUNCH(64, true);
    else
        ATX_GREC_LAUNCH(64, false);
#undef ATX_GREC_LAUNCH
    return ATX_OK;
}

}  // extern "C"
