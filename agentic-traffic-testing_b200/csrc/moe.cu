// Mixture of experts: routing, the plan that sorts (token, choice) pairs by expert, the experts' matrix products over
// their own rows, and the weighted sum.
//   route    soft-max over the router's outputs in fp32; the `top` largest of score + correction are chosen (lowest
//            index on ties), their weight is the plain score times a constant. One warp per token.
//   plan     one CTA: rows per expert, their running offsets, a slot in the sorted order for every pair whose choice is a
//            real expert (choices >= E stand for experts that return their input and take no slot), and the list of
//            (expert, first slot) tiles the products run over. Which slot a pair gets inside its expert's range depends on
//            the order of atomic increments; the arithmetic of a row does not depend on its slot.
//   product  out[slot, :] = A[row(slot), :] W_e^T for the slots of expert e, a tile of 64 slots x 64 outputs per CTA; CTAs
//            past the plan's tile count leave at once, so the launch needs no count on the host. bf16 on the tensor cores
//            (mma.sync m16n8k16, fp32 accumulation), fp32 on the FMA pipe. With `gated`, W_e holds N gate rows then N up
//            rows and the CTA forms silu(gate) * up before it stores.
//   combine  y[t] = shared_gate * y[t] + sum_k w[t, k] * (choice >= E ? x[t] : product[slot(t, k)]).
#include "common.cuh"

#include "../../include/atx_b200.h"

namespace atx {

template <typename XT>
__device__ __forceinline__ float mld(const XT* p, long long i);
template <>
__device__ __forceinline__ float mld<float>(const float* p, long long i) {
    return p[i];
}
template <>
__device__ __forceinline__ float mld<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
    return __bfloat162float(p[i]);
}
__device__ __forceinline__ void mst(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void mst(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

static void set_pdl_moe(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int flags) {
    if (flags & ATX_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
}

constexpr int kRouteMax = 16;   // router outputs per lane: up to 512 outputs

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ correction, int R, int top,
                 float scale, int* __restrict__ sel, float* __restrict__ wgt, int T, int normalize) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long t = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
    if (t >= T) return;
    const float* z = logits + t * ld;
    float s[kRouteMax], c[kRouteMax];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kRouteMax; ++i) {
        const int e = lane + 32 * i;
        s[i] = e < R ? z[e] : -INFINITY;
        mx = fmaxf(mx, s[i]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kRouteMax; ++i) {
        const int e = lane + 32 * i;
        s[i] = e < R ? expf(s[i] - mx) : 0.f;
        sum += s[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < kRouteMax; ++i) {
        const int e = lane + 32 * i;
        s[i] *= inv;
        c[i] = e < R ? s[i] + (correction ? correction[e] : 0.f) : -INFINITY;
    }
    float chosen = 0.f;   // sum of the chosen scores
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY, bs = 0.f;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kRouteMax; ++i) {
            const int e = lane + 32 * i;
            if (c[i] > best) best = c[i], bi = e, bs = s[i];   // ascending e inside a lane: the lowest index wins ties
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            const float os = __shfl_xor_sync(0xffffffffu, bs, o);
            if (ob > best || (ob == best && oi < bi)) best = ob, bi = oi, bs = os;
        }
#pragma unroll
        for (int i = 0; i < kRouteMax; ++i)
            if (lane + 32 * i == bi) c[i] = -INFINITY;
        chosen += bs;
        if (lane == 0) {
            sel[t * top + k] = bi;
            wgt[t * top + k] = normalize ? bs : bs * scale;
        }
    }
    if (normalize && lane == 0) {   // weights = chosen scores divided by their sum, times scale
        const float inv_c = 1.f / (chosen + 1e-20f);
        for (int k = 0; k < top; ++k) wgt[t * top + k] = wgt[t * top + k] * inv_c * scale;
    }
}

// tiles: [0] = number of tiles, then (expert, first slot) pairs from index 2 on.
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ sel, int n_pairs, int E, int tile_rows, int* __restrict__ seg_off,
                int* __restrict__ perm, int* __restrict__ slot_of, int* __restrict__ tiles) {
    extern __shared__ int sh[];   // counts [E] | cursors [E] | tile offsets [E + 1]
    int* cnt = sh;
    int* cur = sh + E;
    int* toff = sh + 2 * E;
    pdl_launch_dependents();
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    pdl_wait();
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = sel[i];
        if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int off = 0, nt = 0;
        for (int e = 0; e < E; ++e) {
            seg_off[e] = off;
            cur[e] = off;
            toff[e] = nt;
            off += cnt[e];
            nt += (cnt[e] + tile_rows - 1) / tile_rows;
        }
        seg_off[E] = off;
        toff[E] = nt;
        tiles[0] = nt;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int n = toff[e + 1] - toff[e];
        for (int j = 0; j < n; ++j) {
            tiles[2 + 2 * (toff[e] + j)] = e;
            tiles[3 + 2 * (toff[e] + j)] = seg_off[e] + j * tile_rows;
        }
    }
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = sel[i];
        int slot = -1;
        if (e >= 0 && e < E) {
            slot = atomicAdd(&cur[e], 1);
            perm[slot] = i;
        }
        slot_of[i] = slot;
    }
}

constexpr int kET = 64, kEK = 64, kELD = kEK + 8, kEStages = 3;

__device__ __forceinline__ void moe_cp16(void* smem_dst, const void* gsrc, bool valid) {
    const uint32_t sz = valid ? 16u : 0u;   // source size 0: sixteen bytes of zeros, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(sz) : "memory");
}

// bf16, tensor cores. A row of slot p: A[(gather ? perm[p] / top : p) * lda]. GATED: two accumulator sets (gate, up);
// the gate row of output n is row n of the expert's matrix and its up row N + n, or, with `interleaved`, rows
// 128 (n / 64) + n % 64 and 64 further (the layout of the tcgen05 GEMM's gated epilogue). Tiles of 64 reduction
// elements arrive by cp.async into three stages, two in flight while one is multiplied: with one or two rows per expert
// (decoded tokens) the kernel only streams the chosen experts' matrices, and what bounds it is bytes in flight.
// BM: slots per tile, 64 or 16. Decode-sized steps have one or two rows per expert; with 16-slot tiles a stage holds a third
// less, three CTAs instead of two fit an SM, and the grid (tiles x output blocks) fits one wave.
template <bool GATED, int BM>
__global__ void __launch_bounds__(128)
moe_gemm_tc_kernel(const __nv_bfloat16* __restrict__ A, long long lda, const int* __restrict__ perm, int top, int gather,
                   const __nv_bfloat16* __restrict__ W, long long expert_stride, long long ldw, void* __restrict__ out,
                   long long ldo, int N, int K, const int* __restrict__ seg_off, const int* __restrict__ tiles,
                   int interleaved) {
    constexpr int NW = GATED ? 2 : 1;
    constexpr int kStageElems = (BM + NW * kET) * kELD;
    extern __shared__ __align__(16) unsigned char moe_smem[];
    __nv_bfloat16* stages = reinterpret_cast<__nv_bfloat16*>(moe_smem);
    __shared__ long long arow[BM];
    pdl_launch_dependents();
    pdl_wait();
    if (static_cast<int>(blockIdx.y) >= tiles[0]) return;
    const int e = tiles[2 + 2 * blockIdx.y], p0 = tiles[3 + 2 * blockIdx.y];
    const int rows = min(BM, seg_off[e + 1] - p0);
    const int n0 = blockIdx.x * kET;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const __nv_bfloat16* We = W + static_cast<long long>(e) * expert_stride;
    const long long g_base = (GATED && interleaved) ? 2ll * n0 : n0;          // matrix row of the tile's first gate output
    const long long u_base = (GATED && interleaved) ? 2ll * n0 + 64 : static_cast<long long>(N) + n0;
    if (threadIdx.x < BM) {
        const int p = p0 + threadIdx.x;
        arow[threadIdx.x] = threadIdx.x < rows ? static_cast<long long>(gather ? perm[p] / top : p) * lda : -1;
    }
    __syncthreads();
    float acc[NW][kET / 8][4];
#pragma unroll
    for (int g = 0; g < NW; ++g)
#pragma unroll
        for (int i = 0; i < kET / 8; ++i) acc[g][i][0] = acc[g][i][1] = acc[g][i][2] = acc[g][i][3] = 0.f;
    const bool vec = (K & 7) == 0 && ((lda | ldw | expert_stride) & 7) == 0 &&
                     ((reinterpret_cast<unsigned long long>(A) | reinterpret_cast<unsigned long long>(W)) & 15) == 0;
    const int nk = (K + kEK - 1) / kEK;
    const int rb = warp;   // a warp owns 16 rows and all 64 outputs of the tile
    auto load = [&](int kc, int stage) {
        __nv_bfloat16* sa = stages + stage * kStageElems;
        __nv_bfloat16* sw = sa + BM * kELD;
        const int k0 = kc * kEK;
        if (vec) {
            for (int c = threadIdx.x; c < kET * (kEK / 8); c += 128) {
                const int r = c / (kEK / 8), k8 = (c - r * (kEK / 8)) * 8;
                const int k = k0 + k8, n = n0 + r;
                const bool w_ok = n < N && k < K;
                if (r < BM) {
                    const bool a_ok = arow[r] >= 0 && k < K;
                    moe_cp16(sa + r * kELD + k8, A + (a_ok ? arow[r] + k : 0), a_ok);
                }
                moe_cp16(sw + r * kELD + k8, We + (w_ok ? (g_base + r) * ldw + k : 0), w_ok);
                if (GATED) moe_cp16(sw + (kET + r) * kELD + k8, We + (w_ok ? (u_base + r) * ldw + k : 0), w_ok);
            }
        } else {
            const __nv_bfloat16 zero = __float2bfloat16_rn(0.f);
            for (int c = threadIdx.x; c < kET * kEK; c += 128) {
                const int r = c / kEK, kk = c - r * kEK;
                const int k = k0 + kk, n = n0 + r;
                if (r < BM) sa[r * kELD + kk] = (arow[r] >= 0 && k < K) ? A[arow[r] + k] : zero;
                sw[r * kELD + kk] = (n < N && k < K) ? We[(g_base + r) * ldw + k] : zero;
                if (GATED) sw[(kET + r) * kELD + kk] = (n < N && k < K) ? We[(u_base + r) * ldw + k] : zero;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (int s = 0; s < kEStages - 1; ++s) {
        if (s < nk) load(s, s);
        else asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int kc = 0; kc < nk; ++kc) {
        asm volatile("cp.async.wait_group %0;" ::"n"(kEStages - 2) : "memory");
        __syncthreads();   // chunk kc has landed for every thread, and the stage chunk kc - 1 used is free
        if (kc + kEStages - 1 < nk) load(kc + kEStages - 1, (kc + kEStages - 1) % kEStages);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        const __nv_bfloat16* sa = stages + (kc % kEStages) * kStageElems;
        const __nv_bfloat16* sw = sa + BM * kELD;
        if (rb * 16 < rows) {
#pragma unroll
            for (int ks = 0; ks < kEK / 16; ++ks) {
                uint32_t a[4];
                ldsm_x4(smem_u32(sa + (rb * 16 + (lane & 15)) * kELD + ks * 16 + (lane >> 4) * 8), a[0], a[1], a[2], a[3]);
#pragma unroll
                for (int g = 0; g < NW; ++g) {
#pragma unroll
                    for (int nb2 = 0; nb2 < kET / 16; ++nb2) {
                        uint32_t b0, b1, b2, b3;
                        ldsm_x4(smem_u32(sw + (g * kET + nb2 * 16 + (lane >> 4) * 8 + (lane & 7)) * kELD + ks * 16 +
                                         ((lane >> 3) & 1) * 8), b0, b1, b2, b3);
                        mma_bf16(acc[g][2 * nb2], a, b0, b1);
                        mma_bf16(acc[g][2 * nb2 + 1], a, b2, b3);
                    }
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int r = rb * 16 + (lane >> 2) + 8 * rr;
        if (r >= rows) continue;
        const long long p = p0 + r;
#pragma unroll
        for (int nb = 0; nb < kET / 8; ++nb) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int n = n0 + nb * 8 + (lane & 3) * 2 + q;
                if (n >= N) continue;
                if (GATED) {
                    const float g = acc[0][nb][2 * rr + q], u = acc[NW - 1][nb][2 * rr + q];
                    reinterpret_cast<__nv_bfloat16*>(out)[p * ldo + n] = __float2bfloat16_rn(g / (1.f + expf(-g)) * u);
                } else {
                    reinterpret_cast<float*>(out)[p * ldo + n] = acc[0][nb][2 * rr + q];
                }
            }
        }
    }
}

// Any element type on the FMA pipe: 64 slots x 64 outputs per CTA, 4 x 4 per thread, fp32 accumulation in a fixed order.
template <typename XT, bool GATED>
__global__ void __launch_bounds__(256)
moe_gemm_fma_kernel(const XT* __restrict__ A, long long lda, const int* __restrict__ perm, int top, int gather,
                    const XT* __restrict__ W, long long expert_stride, long long ldw, void* __restrict__ out, long long ldo,
                    int N, int K, const int* __restrict__ seg_off, const int* __restrict__ tiles, int interleaved) {
    constexpr int KC = 16;
    __shared__ float sa[KC][kET + 1];
    __shared__ float sw[GATED ? 2 : 1][KC][kET + 1];
    __shared__ long long arow[kET];
    pdl_launch_dependents();
    pdl_wait();
    if (static_cast<int>(blockIdx.y) >= tiles[0]) return;
    const int e = tiles[2 + 2 * blockIdx.y], p0 = tiles[3 + 2 * blockIdx.y];
    const int rows = min(kET, seg_off[e + 1] - p0);
    const int n0 = blockIdx.x * kET;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const XT* We = W + static_cast<long long>(e) * expert_stride;
    const long long g_base = (GATED && interleaved) ? 2ll * n0 : n0;
    const long long u_base = (GATED && interleaved) ? 2ll * n0 + 64 : static_cast<long long>(N) + n0;
    if (threadIdx.x < kET) {
        const int p = p0 + threadIdx.x;
        arow[threadIdx.x] = static_cast<int>(threadIdx.x) < rows ? static_cast<long long>(gather ? perm[p] / top : p) * lda : -1;
    }
    __syncthreads();
    float acc[GATED ? 2 : 1][4][4];
#pragma unroll
    for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[g][i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += KC) {
        for (int c = threadIdx.x; c < kET * KC; c += 256) {
            const int r = c / KC, kk = c - r * KC;
            const int k = k0 + kk, n = n0 + r;
            sa[kk][r] = (arow[r] >= 0 && k < K) ? mld(A, arow[r] + k) : 0.f;
            sw[0][kk][r] = (n < N && k < K) ? mld(We, (g_base + r) * ldw + k) : 0.f;
            if (GATED) sw[GATED ? 1 : 0][kk][r] = (n < N && k < K) ? mld(We, (u_base + r) * ldw + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < KC; ++kk) {
            float av[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
            for (int g = 0; g < (GATED ? 2 : 1); ++g) {
                float bv[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) bv[j] = sw[g][kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[g][i][j] = fmaf(av[i], bv[j], acc[g][i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= rows) continue;
        const long long p = p0 + r;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            if (GATED) {
                const float g = acc[0][i][j], u = acc[GATED ? 1 : 0][i][j];
                mst(reinterpret_cast<XT*>(out), p * ldo + n, g / (1.f + expf(-g)) * u);
            } else {
                reinterpret_cast<float*>(out)[p * ldo + n] = acc[0][i][j];
            }
        }
    }
}

// out[slot, :] = x[perm[slot] / top, :] for every slot the plan handed out: the rows of each expert back to back, so that
// a GEMM whose operands arrive by TMA can read them as tiles.
template <typename XT>
__global__ void __launch_bounds__(128)
moe_gather_rows_kernel(const XT* __restrict__ x, long long ldx, const int* __restrict__ perm, int top,
                       const int* __restrict__ seg_off, int E, XT* __restrict__ out, long long ldo, int W) {
    pdl_launch_dependents();
    pdl_wait();
    const long long slot = blockIdx.x;
    if (slot >= seg_off[E]) return;
    const XT* src = x + static_cast<long long>(perm[slot] / top) * ldx;
    XT* dst = out + slot * ldo;
    constexpr int PER = 16 / sizeof(XT);
    if (W % PER == 0 && ldx % PER == 0 && ldo % PER == 0 &&
        ((reinterpret_cast<unsigned long long>(x) | reinterpret_cast<unsigned long long>(out)) & 15) == 0) {
        for (int i = threadIdx.x; i < W / PER; i += blockDim.x)
            reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
        return;
    }
    for (int i = threadIdx.x; i < W; i += blockDim.x) dst[i] = src[i];
}

template <typename XT>
__global__ void __launch_bounds__(256)
moe_combine_kernel(float* __restrict__ y, const float* __restrict__ ye, long long lde, const XT* __restrict__ x,
                   const int* __restrict__ sel, const float* __restrict__ wgt, const int* __restrict__ slot_of,
                   const float* __restrict__ shared_gate, long long ldsg, int W, int top, int E) {
    __shared__ float s_w[64];
    __shared__ long long s_row[64];   // row of ye, or -1: the choice returns the input
    pdl_launch_dependents();
    pdl_wait();
    const long long t = blockIdx.x;
    for (int k = threadIdx.x; k < top; k += blockDim.x) {
        s_w[k] = wgt[t * top + k];
        s_row[k] = sel[t * top + k] >= E ? -1 : static_cast<long long>(slot_of[t * top + k]) * lde;
    }
    const float sg = shared_gate ? 1.f / (1.f + expf(-shared_gate[t * ldsg])) : 0.f;
    __syncthreads();
    float* yr = y + t * W;
    const XT* xr = x + t * W;
    if ((W & 3) == 0 && (lde & 3) == 0 &&
        ((reinterpret_cast<unsigned long long>(y) | reinterpret_cast<unsigned long long>(ye) |
          reinterpret_cast<unsigned long long>(x)) & 15) == 0) {
        for (int i = threadIdx.x; i < W / 4; i += blockDim.x) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            if (shared_gate) {
                const float4 v = reinterpret_cast<const float4*>(yr)[i];
                acc = make_float4(sg * v.x, sg * v.y, sg * v.z, sg * v.w);
            }
            float4 xin = make_float4(0.f, 0.f, 0.f, 0.f);
            bool have_x = false;
            for (int k = 0; k < top; ++k) {
                float4 v;
                if (s_row[k] < 0) {
                    if (!have_x) {
                        xin = make_float4(mld(xr, 4 * i), mld(xr, 4 * i + 1), mld(xr, 4 * i + 2), mld(xr, 4 * i + 3));
                        have_x = true;
                    }
                    v = xin;
                } else {
                    v = *reinterpret_cast<const float4*>(ye + s_row[k] + 4 * i);
                }
                const float w = s_w[k];
                acc.x = fmaf(w, v.x, acc.x), acc.y = fmaf(w, v.y, acc.y), acc.z = fmaf(w, v.z, acc.z), acc.w = fmaf(w, v.w, acc.w);
            }
            reinterpret_cast<float4*>(yr)[i] = acc;
        }
        return;
    }
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float acc = shared_gate ? sg * yr[i] : 0.f;
        for (int k = 0; k < top; ++k) acc = fmaf(s_w[k], s_row[k] < 0 ? mld(xr, i) : ye[s_row[k] + i], acc);
        yr[i] = acc;
    }
}

}  // namespace atx

using namespace atx;

extern "C" {

int atx_moe_route(const float* logits, long long ld, const float* correction, int R, int top, float scale, int* sel,
                  float* wgt, int T, int flags, atx_stream_t stream) {
    return atx_moe_route_opts(logits, ld, correction, R, top, scale, 0, sel, wgt, T, flags, stream);
}

int atx_moe_route_opts(const float* logits, long long ld, const float* correction, int R, int top, float scale,
                       int normalize, int* sel, float* wgt, int T, int flags, atx_stream_t stream) {
    ATX_REQUIRE(logits && sel && wgt, "atx_moe_route: null pointer");
    ATX_REQUIRE(T > 0 && R > 0 && R <= 32 * kRouteMax && top > 0 && top <= R && ld >= R,
                "atx_moe_route: bad shape T=%d outputs=%d (<= %d) top=%d ld=%lld", T, R, 32 * kRouteMax, top, ld);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3((T + 3) / 4);
    cfg.blockDim = dim3(128);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl_moe(cfg, attr, flags);
    ATX_CUDA(cudaLaunchKernelEx(&cfg, moe_route_kernel, logits, ld, correction, R, top, scale, sel, wgt, T, normalize));
    return ATX_OK;
}

int atx_moe_tile_rows(void) { return kET; }

int atx_moe_plan(const int* sel, int n_pairs, int E, int tile_rows, int* seg_off, int* perm, int* slot_of, int* tiles,
                 int flags, atx_stream_t stream) {
    ATX_REQUIRE(sel && seg_off && perm && slot_of && tiles, "atx_moe_plan: null pointer");
    ATX_REQUIRE(n_pairs > 0 && E > 0 && E <= 4096 && tile_rows > 0, "atx_moe_plan: bad shape pairs=%d experts=%d tile=%d",
                n_pairs, E, tile_rows);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(1024);
    cfg.dynamicSmemBytes = sizeof(int) * (3 * static_cast<size_t>(E) + 1);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl_moe(cfg, attr, flags);
    ATX_CUDA(cudaLaunchKernelEx(&cfg, moe_plan_kernel, sel, n_pairs, E, tile_rows, seg_off, perm, slot_of, tiles));
    return ATX_OK;
}

int atx_moe_expert_gemm(const void* A, long long lda, const int* perm, int top, int gather, const void* W,
                        long long expert_stride, long long ldw, void* out, long long ldo, int N, int K, int gated,
                        int interleaved, int tile_rows, const int* seg_off, const int* tiles, int max_tiles, int dtype,
                        int flags, atx_stream_t stream) {
    ATX_REQUIRE(A && W && out && seg_off && tiles && (!gather || perm), "atx_moe_expert_gemm: null pointer");
    ATX_REQUIRE(N > 0 && K > 0 && max_tiles > 0 && max_tiles <= 65535 && top > 0 && ldw >= K && lda >= K && ldo >= N,
                "atx_moe_expert_gemm: bad shape N=%d K=%d tiles=%d lda=%lld ldw=%lld ldo=%lld", N, K, max_tiles, lda, ldw, ldo);
    ATX_REQUIRE(!interleaved || (gated && N % 64 == 0), "atx_moe_expert_gemm: interleaved gate / up rows need N %% 64 == 0");
    ATX_REQUIRE(tile_rows == kET || (tile_rows == 16 && dtype == ATX_DT_BF16),
                "atx_moe_expert_gemm: tiles of %d slots (64, or 16 for bf16)", tile_rows);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3((N + kET - 1) / kET, max_tiles);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl_moe(cfg, attr, flags);
#define ATX_MOE_LAUNCH(KERNEL_, T_)                                                                                     \
    ATX_CUDA(cudaLaunchKernelEx(&cfg, KERNEL_, reinterpret_cast<const T_*>(A), lda, perm, top, gather,                \
                                reinterpret_cast<const T_*>(W), expert_stride, ldw, out, ldo, N, K, seg_off, tiles,  \
                                interleaved))
    if (dtype == ATX_DT_BF16) {
        cfg.blockDim = dim3(128);
        const int smem = kEStages * ((tile_rows + (gated ? 2 : 1) * kET) * kELD) * 2;
        cfg.dynamicSmemBytes = smem;
        static bool attr_done[4] = {false, false, false, false};
        const int which = (gated ? 1 : 0) + (tile_rows == 16 ? 2 : 0);
#define ATX_MOE_TC(G_, BM_)                                                                                              \
    do {                                                                                                                 \
        if (!attr_done[which]) {                                                                                         \
            ATX_CUDA(cudaFuncSetAttribute(moe_gemm_tc_kernel<G_, BM_>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); \
            attr_done[which] = true;                                                                                     \
        }                                                                                                                \
        ATX_MOE_LAUNCH((moe_gemm_tc_kernel<G_, BM_>), __nv_bfloat16);                                                    \
    } while (0)
        if (gated && tile_rows == 16) ATX_MOE_TC(true, 16);
        else if (gated) ATX_MOE_TC(true, 64);
        else if (tile_rows == 16) ATX_MOE_TC(false, 16);
        else ATX_MOE_TC(false, 64);
#undef ATX_MOE_TC
    } else {
        cfg.blockDim = dim3(256);
        if (gated)
            ATX_MOE_LAUNCH((moe_gemm_fma_kernel<float, true>), float);
        else
            ATX_MOE_LAUNCH((moe_gemm_fma_kernel<float, false>), float);
    }
#undef ATX_MOE_LAUNCH
    return ATX_OK;
}

int atx_moe_gather_rows(const void* x, long long ldx, const int* perm, int top, const int* seg_off, int E, void* out,
                        long long ldo, int max_slots, int W, int dtype, int flags, atx_stream_t stream) {
    ATX_REQUIRE(x && perm && seg_off && out, "atx_moe_gather_rows: null pointer");
    ATX_REQUIRE(max_slots > 0 && W > 0 && top > 0 && E > 0 && ldx >= W && ldo >= W, "atx_moe_gather_rows: bad shape slots=%d W=%d",
                max_slots, W);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(max_slots);
    cfg.blockDim = dim3(128);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl_moe(cfg, attr, flags);
    if (dtype == ATX_DT_F32)
        ATX_CUDA(cudaLaunchKernelEx(&cfg, moe_gather_rows_kernel<float>, reinterpret_cast<const float*>(x), ldx, perm, top,
                                    seg_off, E, reinterpret_cast<float*>(out), ldo, W));
    else
        ATX_CUDA(cudaLaunchKernelEx(&cfg, moe_gather_rows_kernel<__nv_bfloat16>, reinterpret_cast<const __nv_bfloat16*>(x), ldx,
                                    perm, top, seg_off, E, reinterpret_cast<__nv_bfloat16*>(out), ldo, W));
    return ATX_OK;
}

int atx_moe_combine(float* y, const float* ye, long long lde, const void* x, const int* sel, const float* wgt,
                    const int* slot_of, const float* shared_gate, long long ldsg, int T, int W, int top, int E, int dtype,
                    int flags, atx_stream_t stream) {
    ATX_REQUIRE(y && ye && x && sel && wgt && slot_of, "atx_moe_combine: null pointer");
    ATX_REQUIRE(T > 0 && W > 0 && top > 0 && top <= 64 && E > 0 && lde >= W, "atx_moe_combine: bad shape T=%d W=%d top=%d (<= 64)",
                T, W, top);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(T);
    cfg.blockDim = dim3(256);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    set_pdl_moe(cfg, attr, flags);
    if (dtype == ATX_DT_F32)
        ATX_CUDA(cudaLaunchKernelEx(&cfg, moe_combine_kernel<float>, y, ye, lde, reinterpret_cast<const float*>(x), sel, wgt,
                                    slot_of, shared_gate, ldsg, W, top, E));
    else
        ATX_CUDA(cudaLaunchKernelEx(&cfg, moe_combine_kernel<__nv_bfloat16>, y, ye, lde,
                                    reinterpret_cast<const __nv_bfloat16*>(x), sel, wgt, slot_of, shared_gate, ldsg, W, top, E));
    return ATX_OK;
}

}  // extern "C"
