// The recurrence with a decay per key channel (seqmix.cu, atx_gated_linear_recurrence) for prompt portions, in a
// chunk-parallel form on the tensor cores.
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T,   y_t = S_t^T (s q_t),   a_t[d] = exp(g_t[d]), g <= 0 given          (S: D x V, fp32)
//
// Over a chunk of 16 consecutive tokens with b_t[d] = sum_{u <= t} g_u[d] (inside the chunk) and S_in the state before it:
//
//   y_t   = S_in^T (s q_t * e^{b_t})  +  sum_{j <= t} (sum_d s q_t[d] k_j[d] e^{b_t[d] - b_j[d]}) v_j
//   S_out = diag(e^{b_last}) S_in     +  sum_j (k_j * e^{b_last - b_j}) v_j^T
//
// Every exponent is a sum of g over a range of tokens, hence <= 0: nothing overflows however strong a decay is, and a factor
// that underflows stands for a term that has vanished. The pair weights of the middle sum carry a different decay in every
// key channel, so they do not factor into a product of a query-side and a key-side matrix with bounded entries; a chunk is
// short enough to evaluate them as they stand: 136 pairs x D exponentials in fp32 on the FMA / MUFU pipes. The three
// matrix products (state read-out, pair weights times values, state update) run on mma.sync m16n8k16 with bf16 operands
// and fp32 accumulation. What stays fp32: the state (it lives in accumulator registers for the whole portion and is read
// out as a bf16 high part plus a bf16 remainder), the logarithms, their running sums, every exponential, and the pair
// weights until the one rounding to bf16 that a tensor-core operand gets.
//
// One CTA = one sequence x one head x 128 value columns, eight warps of 16 value columns each. The state tile is kept
// TRANSPOSED (rows = value columns, columns = key channels) so that its accumulator fragments turn into A fragments of
// S^T Q^T in registers. The next chunk's rows are fetched into registers while this chunk's products run. Sequences are
// walked as in seqmix.cu: rows [seq_start, seq_start + seq_count), state slot seq_slot, zero state when seq_pos0 == 0.
#include "common.cuh"

#include "../../include/atx_b200.h"

namespace atx {

constexpr int kGcC = 16;    // tokens per chunk
constexpr int kGcV = 128;   // value columns per CTA
constexpr int kGcT = 256;   // threads per CTA

template <int D>
__global__ void __launch_bounds__(kGcT, D > 64 ? 1 : 2)
gla_chunked_kernel(const float* __restrict__ q, long long ldq, const float* __restrict__ k, long long ldk,
                   const float* __restrict__ v, long long ldv, const float* __restrict__ ldecay, long long ldc, int H, int V,
                   float qscale, float* __restrict__ state, float* __restrict__ y, long long ldy,
                   const int* __restrict__ seq_start, const int* __restrict__ seq_count, const int* __restrict__ seq_pos0,
                   const int* __restrict__ seq_slot) {
    constexpr int LQ = D + 8, LV = kGcV + 8, LA = kGcC + 8;   // padded rows: ldmatrix without bank conflicts
    constexpr int NQ = kGcC * D / kGcT, NV = kGcC * kGcV / kGcT;
    __shared__ __align__(16) __nv_bfloat16 sQ[kGcC * LQ];     // s q_t e^{b_t}
    __shared__ __align__(16) __nv_bfloat16 sK[kGcC * LQ];     // k_j e^{b_last - b_j}
    __shared__ __align__(16) __nv_bfloat16 sV[kGcC * LV];     // v_j
    __shared__ __align__(16) __nv_bfloat16 sA[kGcC * LA];     // pair weights, j <= t
    __shared__ float fq[kGcC * D], fk[kGcC * D], fb[kGcC * D];   // s q, k, and g then its running sums b
    __shared__ float sE[D];                                       // e^{b_last}
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * kGcV;
    const int n = seq_count[s];
    if (n <= 0) return;
    const long long r0 = seq_start[s];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int vw = warp * 16;
    const int vr = v0 + vw + (lane >> 2);        // value column of accumulator elements 0, 1 (elements 2, 3: + 8)
    const int c2 = 2 * (lane & 3);               // first of this thread's two columns inside an 8-wide tile

    float S[D / 8][4];
    float* st = state + (static_cast<long long>(seq_slot[s]) * H + h) * D * V;
    const bool fresh = seq_pos0[s] == 0;
#pragma unroll
    for (int nd = 0; nd < D / 8; ++nd)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int vv = vr + 8 * (e >> 1), d = nd * 8 + c2 + (e & 1);
            S[nd][e] = (!fresh && vv < V) ? st[static_cast<long long>(d) * V + vv] : 0.f;
        }
    for (int e = threadIdx.x; e < kGcC * LA; e += kGcT) sA[e] = __float2bfloat16_rn(0.f);   // keys after the query stay 0

    float rq[NQ], rk[NQ], rg[NQ], rv[NV];
    auto fetch = [&](int c0) {   // rows past the portion: nothing to add, no decay
        const int cn = min(kGcC, n - c0);
#pragma unroll
        for (int u = 0; u < NQ; ++u) {
            const int e = threadIdx.x + u * kGcT, i = e / D, d = e - i * D;
            rq[u] = rk[u] = rg[u] = 0.f;
            if (i < cn) {
                const long long row = r0 + c0 + i;
                rq[u] = q[row * ldq + static_cast<long long>(h) * D + d];
                rk[u] = k[row * ldk + static_cast<long long>(h) * D + d];
                rg[u] = ldecay[row * ldc + static_cast<long long>(h) * D + d];
            }
        }
#pragma unroll
        for (int u = 0; u < NV; ++u) {
            const int e = threadIdx.x + u * kGcT, i = e / kGcV, j = e - i * kGcV;
            rv[u] = (i < cn && v0 + j < V) ? v[(r0 + c0 + i) * ldv + static_cast<long long>(h) * V + v0 + j] : 0.f;
        }
    };
    fetch(0);

    for (int c0 = 0; c0 < n; c0 += kGcC) {
        const int cn = min(kGcC, n - c0);
        __syncthreads();   // the previous chunk's tiles have been consumed
#pragma unroll
        for (int u = 0; u < NQ; ++u) {
            const int e = threadIdx.x + u * kGcT;
            fq[e] = rq[u] * qscale;
            fk[e] = rk[u];
            fb[e] = rg[u];
        }
#pragma unroll
        for (int u = 0; u < NV; ++u) {
            const int e = threadIdx.x + u * kGcT, i = e / kGcV, j = e - i * kGcV;
            sV[i * LV + j] = __float2bfloat16_rn(rv[u]);
        }
        __syncthreads();
        if (c0 + kGcC < n) fetch(c0 + kGcC);   // in flight while this chunk is worked on
        if (threadIdx.x < D) {                  // running sums of the logarithms down the chunk, per key channel
            float b = 0.f;
#pragma unroll
            for (int i = 0; i < kGcC; ++i) {
                b += fb[i * D + threadIdx.x];
                fb[i * D + threadIdx.x] = b;
            }
            sE[threadIdx.x] = expf(b);
        }
        __syncthreads();
        // operands of the read-out and of the update
#pragma unroll
        for (int u = 0; u < NQ; ++u) {
            const int e = threadIdx.x + u * kGcT, i = e / D, d = e - i * D;
            const float b = fb[e];
            sQ[i * LQ + d] = __float2bfloat16_rn(fq[e] * expf(b));
            sK[i * LQ + d] = __float2bfloat16_rn(fk[e] * expf(fb[(kGcC - 1) * D + d] - b));
        }
        // pair weights inside the chunk, as they stand: a warp per pair, its lanes over the key channels
        for (int p = warp; p < kGcC * (kGcC + 1) / 2; p += kGcT / 32) {
            int t = 0, rem = p;
            while (rem > t) {   // pair p = (t, j) with j <= t, rows of the lower triangle back to back
                rem -= t + 1;
                ++t;
            }
            const int j = rem;
            if (t >= cn) continue;   // rows past the portion: their weights stay what they were and are never read as rows < cn
            float a = 0.f;
#pragma unroll
            for (int d = lane; d < D; d += 32)
                a = fmaf(fq[t * D + d] * fk[j * D + d], expf(fb[t * D + d] - fb[j * D + d]), a);
            a = warp_sum(a);
            if (lane == 0) sA[t * LA + j] = __float2bfloat16_rn(a);
        }
        __syncthreads();

        // ---- Y^T (this warp's 16 value columns x 16 tokens) = S_in^T Q^T + V^T A^T -------------------------------------
        float acc[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        if (!(fresh && c0 == 0)) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                uint32_t ah[4], al[4];
#pragma unroll
                for (int f = 0; f < 4; ++f) {
                    const float x0 = S[2 * kk + (f >> 1)][2 * (f & 1)], x1 = S[2 * kk + (f >> 1)][2 * (f & 1) + 1];
                    ah[f] = pack_bf16(x0, x1);
                    al[f] = pack_bf16(x0 - bf16lo(ah[f]), x1 - bf16hi(ah[f]));
                }
                uint32_t b0, b1, b2, b3;
                ldsm_x4(smem_u32(sQ + ((lane >> 4) * 8 + (lane & 7)) * LQ + kk * 16 + ((lane >> 3) & 1) * 8), b0, b1, b2, b3);
                mma_bf16(acc[0], ah, b0, b1);
                mma_bf16(acc[1], ah, b2, b3);
                mma_bf16(acc[0], al, b0, b1);
                mma_bf16(acc[1], al, b2, b3);
            }
        }
        uint32_t av[4];   // V^T: 16 value columns x 16 tokens, the A operand of the two products that follow
        ldsm_x4_t(smem_u32(sV + ((lane >> 4) * 8 + (lane & 7)) * LV + vw + ((lane >> 3) & 1) * 8), av[0], av[1], av[2], av[3]);
        {
            uint32_t b0, b1, b2, b3;
            ldsm_x4(smem_u32(sA + ((lane >> 4) * 8 + (lane & 7)) * LA + ((lane >> 3) & 1) * 8), b0, b1, b2, b3);
            mma_bf16(acc[0], av, b0, b1);
            mma_bf16(acc[1], av, b2, b3);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int t = i * 8 + c2 + (e & 1), vv = vr + 8 * (e >> 1);
                if (t < cn && vv < V) y[(r0 + c0 + t) * ldy + static_cast<long long>(h) * V + vv] = acc[i][e];
            }

        // ---- the state after the chunk: S^T = S^T diag(e^{b_last}) + V^T K~ ---------------------------------------------
#pragma unroll
        for (int nd = 0; nd < D / 8; ++nd) {
            const float e0 = sE[nd * 8 + c2], e1 = sE[nd * 8 + c2 + 1];
            S[nd][0] *= e0;
            S[nd][1] *= e1;
            S[nd][2] *= e0;
            S[nd][3] *= e1;
        }
#pragma unroll
        for (int nb2 = 0; nb2 < D / 16; ++nb2) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(smem_u32(sK + (((lane >> 3) & 1) * 8 + (lane & 7)) * LQ + nb2 * 16 + (lane >> 4) * 8), b0, b1, b2, b3);
            mma_bf16(S[2 * nb2], av, b0, b1);
            mma_bf16(S[2 * nb2 + 1], av, b2, b3);
        }
    }
#pragma unroll
    for (int nd = 0; nd < D / 8; ++nd)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int vv = vr + 8 * (e >> 1), d = nd * 8 + c2 + (e & 1);
            if (vv < V) st[static_cast<long long>(d) * V + vv] = S[nd][e];
        }
}

template <int D>
static int launch_gla_chunked(const float* q, long long ldq, const float* k, long long ldk, const float* v, long long ldv,
                              const float* ldecay, long long ldc, int H, int V, float qscale, float* state, float* y,
                              long long ldy, const int* seq_start, const int* seq_count, const int* seq_pos0,
                              const int* seq_slot, int n_seqs, int flags, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(n_seqs, H, (V + kGcV - 1) / kGcV);
    cfg.blockDim = dim3(kGcT);
    cfg.stream = stream;
    if (flags & ATX_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    ATX_CUDA(cudaLaunchKernelEx(&cfg, gla_chunked_kernel<D>, q, ldq, k, ldk, v, ldv, ldecay, ldc, H, V, qscale, state, y, ldy,
                                seq_start, seq_count, seq_pos0, seq_slot));
    return ATX_OK;
}

}  // namespace atx

using namespace atx;

extern "C" {

int atx_gated_linear_recurrence_chunked_supported(int D) { return (D == 32 || D == 64 || D == 96 || D == 128) ? 1 : 0; }

int atx_gated_linear_recurrence_chunked(const float* q, long long ldq, const float* k, long long ldk, const float* v,
                                        long long ldv, const float* ldecay, long long ldc, int H, int D, int V, float qscale,
                                        float* state, float* y, long long ldy, const int* seq_start, const int* seq_count,
                                        const int* seq_pos0, const int* seq_slot, int n_seqs, int flags,
                                        atx_stream_t stream) {
    ATX_REQUIRE(q && k && v && ldecay && state && y && seq_start && seq_count && seq_pos0 && seq_slot,
                "atx_gated_linear_recurrence_chunked: null pointer");
    ATX_REQUIRE(n_seqs > 0 && H > 0 && V > 0 && atx_gated_linear_recurrence_chunked_supported(D),
                "atx_gated_linear_recurrence_chunked: bad shape n_seqs=%d H=%d D=%d V=%d", n_seqs, H, D, V);
    cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
#define ATX_GLA_CASE(D_)                                                                                                  \
    case D_:                                                                                                              \
        return launch_gla_chunked<D_>(q, ldq, k, ldk, v, ldv, ldecay, ldc, H, V, qscale, state, y, ldy, seq_start,        \
                                      seq_count, seq_pos0, seq_slot, n_seqs, flags, cs)
    switch (D) {
        ATX_GLA_CASE(32);
        ATX_GLA_CASE(64);
        ATX_GLA_CASE(96);
        ATX_GLA_CASE(128);
    }
#undef ATX_GLA_CASE
    return ATX_OK;
}

}  // extern "C"
