/* atx_b200 — C ABI of the B200-native Llama inference kernels (libatx_b200.so).
 *
 * The reference (dlamagna/agentic-traffic-testing) has no FFI of its own: its L5 llm-backend calls
 * the third-party engines vLLM (llm/serve_llm.py:374-379, 521-531) and HF transformers
 * (llm/hf_cpu_server.py:39-50, 91). This header is the seam a replacement engine binds beneath
 * `AsyncVLLMBackend.generate` (llm/serve_llm.py:504): each entry point names the reference
 * arithmetic it replaces. All pointers are DEVICE pointers unless stated; every buffer is owned by
 * the caller; calls are asynchronous on `stream`, never synchronise the host and (unless stated)
 * allocate nothing. Return value: 0 on success, negative on error with text in atx_last_error().
 *
 * Numeric conventions: activations entering a GEMM are bf16, the residual stream and GEMM
 * accumulators are fp32, the KV cache is bf16, softmax / norms reduce in fp32.
 * Index conventions: token ids, positions, slots, block tables and lengths are int32.
 */
#ifndef ATX_B200_H
#define ATX_B200_H

#ifdef __cplusplus
extern "C" {
#endif

typedef void* atx_stream_t; /* a cudaStream_t */

#define ATX_VERSION 100

/* error codes */
#define ATX_OK 0
#define ATX_ERR_ARG -1
#define ATX_ERR_CUDA -2
#define ATX_ERR_UNSUPPORTED -3
#define ATX_ERR_LIMIT -4

/* flags */
#define ATX_FLAG_PDL 1 /* launch with programmatic dependent launch (stream serialization) */
/* atx_gemm_run, ATX_GEMM_ADD_F32, T <= 64: sum the K-splits in a FIXED order (the splits of a tile form a
 * thread-block cluster reduced through distributed shared memory, one CTA adds each output element) instead
 * of letting every split race its red.add: results are bit-reproducible run to run; splits become 1/2/4/8. */
#define ATX_FLAG_ORDERED 2
/* atx_rmsnorm only: `add` points to bf16 [T, H] instead of fp32 (a partial projection all-reduced in bf16) */
#define ATX_FLAG_ADD_BF16 4

/* Thread-local text of the last error raised on the calling thread. Never NULL. */
const char* atx_last_error(void);
int atx_version(void);
/* Device facts of the current device (host pointers may be NULL). */
int atx_device_info(int* sm_count, int* cc_major, int* cc_minor);

/* ---- GEMM: out[t, n] (+)= sum_k X[t, k] * W[n, k] -------------------------------------------------
 * Replaces torch.nn.functional.linear in transformers/models/llama/modeling_llama.py:182-184
 * (gate/up/down), :259-289 (q/k/v/o) and :499 (lm_head). W: [N, K] bf16 row-major (HF layout),
 * X: [T_cap, ldx] bf16. A plan caches the TMA descriptors for one (W, X buffer) pair; creating it
 * is host-only work (no device allocation, no launch). T may vary per call (1..T_cap). */
typedef struct atx_gemm_plan atx_gemm_plan;
#define ATX_GEMM_STORE_F32 0  /* out fp32 = acc                                            */
#define ATX_GEMM_ADD_F32 1    /* out fp32 += acc (atomic; enables split-K; fuses residual) */
#define ATX_GEMM_STORE_BF16 2 /* out bf16 = round(acc)                                     */
/* Fused SwiGLU (modeling_llama.py:182-184): W holds gate and up rows INTERLEAVED in groups of 64
 * (rows [128j, 128j+64) = gate[64j..], rows [128j+64, 128j+128) = up[64j..]); out is bf16
 * [T, N/2] with out[t, 64j+i] = silu(acc_gate) * acc_up. Split-K (T <= 64, splits in {2,4,8} dividing
 * K/64) runs the splits of a tile as one thread-block cluster and sums them through distributed shared
 * memory in a fixed order: no workspace, no atomics, repeatable bit for bit. */
#define ATX_GEMM_SWIGLU_BF16 3
/* out bf16 = max(acc, 0)^2: the activation between the GEMMs of a feed-forward without a gate. Split-K (T <= 64) as for
 * SwiGLU: the splits of a tile are one cluster, summed in a fixed order before the activation. */
#define ATX_GEMM_RELU2_BF16 4
/* ATX_GEMM_SWIGLU_BF16 with clamps (same row layout, same split-K): out = g sigmoid(alpha g) (u + shift) with g = min(acc_gate,
 * limit), u = clamp(acc_up, -limit, limit); the constants are the plan's (atx_gemm_plan_set_gate). */
#define ATX_GEMM_GLU_CLAMP_BF16 5
int atx_gemm_plan_create(atx_gemm_plan** plan, const void* W, long long N, long long K, const void* X,
                         long long T_cap, long long ldx);
void atx_gemm_plan_destroy(atx_gemm_plan* plan);
int atx_gemm_plan_set_gate(atx_gemm_plan* plan, float alpha, float limit, float shift);
/* splits: K partitions (>=1); 0 = choose (ADD and SWIGLU modes may split). ldo: out row pitch in elements. */
int atx_gemm_run(const atx_gemm_plan* plan, void* out, long long ldo, int T, int mode, int splits,
                 int flags, atx_stream_t stream);
int atx_gemm_auto_splits(long long N, long long K, int T);
/* The prefill-sized kernel over groups of rows that each have their own block of W (a mixture of experts: W stacks the
 * experts' matrices, n_group rows each; X holds every expert's rows back to back). tiles / seg_off as atx_moe_plan writes
 * them with tile_rows = atx_gemm_grouped_tile_rows(): out[slot, :] = X[slot, :] W_e^T for the slots of expert e. The grid
 * is sized for max_row_tiles; the real count is read on the device. Modes that store (no ADD). */
int atx_gemm_grouped_tile_rows(void);
int atx_gemm_run_grouped(const atx_gemm_plan* plan, void* out, long long ldo, int n_group, int mode, const int* seg_off,
                         const int* tiles, int max_row_tiles, int flags, atx_stream_t stream);

/* ---- embedding gather: out[t, :] = float(table[ids[t], :]) ---------------------------------------
 * Replaces LlamaModel.embed_tokens (modeling_llama.py:375-427). table: [V, H] bf16, out fp32. */
int atx_embed_gather(const int* ids, const void* table, float* out, int T, int H, int V,
                     atx_stream_t stream);

/* ---- RMSNorm: out[t, :] = bf16( w * x[r, :] * rsqrt(mean(x[r, :]^2) + eps) ), r = rows ? rows[t] : t
 * Replaces LlamaRMSNorm.forward (modeling_llama.py:62-67) and, with `add`, the residual add before it
 * (LlamaDecoderLayer.forward :313-332). x fp32 (the residual stream), w bf16, out bf16.
 * add (nullable, fp32 [T, H]): x[r, :] += add[r, :] first; without `rows` the sum is written back to x
 * and add is cleared (tensor parallelism: add = all-reduced partial o_proj / down_proj output). With
 * ATX_FLAG_ADD_BF16, add is bf16 [T, H] and is left as it is.
 * Optionally zero-fills `zero_ptr[0 .. zero_bytes)` (16-byte multiple) for a following split-K GEMM. */
int atx_rmsnorm(float* x, float* add, const int* rows, const void* w, void* out, int T, int H, float eps,
                void* zero_ptr, long long zero_bytes, int flags, atx_stream_t stream);

/* ---- tensor-parallel: all-reduce + residual add + RMSNorm in one kernel over NVLink peer memory -----
 * Replaces the NCCL all-reduce vLLM issues after o_proj / down_proj of a tensor-parallel Llama layer
 * (the reference reaches it through llm/serve_llm.py:374-379) together with the residual add and
 * LlamaRMSNorm that follow (modeling_llama.py:313-332, 62-67). One process per GPU; every rank calls
 * it with the same T. Two forms, both two-shot with rank r owning the token rows t = r (mod world).
 *
 * Flag-barrier form (up to 256 rows).  part_ptrs[p] / flag_ptrs[p] (HOST arrays of `world` device pointers) are
 * rank p's partial-sum buffer [T, H] fp32 and flag array int[2 * world], both mapped into this process (symmetric /
 * IPC memory).  x fp32 is the residual stream, w the bf16 norm weight, `rows` (nullable) gathers rows before
 * the norm.  clear_buf (nullable): the OTHER ping-pong partial buffer of this rank, first clear_rows rows are
 * zeroed after the cross-GPU barrier.  state: int[2] in local device memory, zero-initialised once.
 * zero_ptr / zero_bytes as in atx_rmsnorm.  The rank pulls
 * only its own rows of every peer's partial buffer, keeps the fp32 residual of its own rows in x (rows it does
 * not own go stale: x must not be read whole between calls), and writes the normalised bf16 rows into EVERY
 * rank's activation buffer through out_ptrs[p] (HOST array of `world` peer-mapped device pointers to the same
 * [T, H] bf16 buffer on each rank). A second cross-GPU barrier inside the kernel keeps it running until
 * every peer's rows have arrived here, so the consumer only needs stream order. flag_ptrs[p] must hold
 * int[2 * world]. NVLink bytes per rank: (world-1)/world * T*H*6. */
int atx_reduce_scatter_rmsnorm_all_gather(float* x, const void* const* part_ptrs, void* const* flag_ptrs,
                                          void* const* out_ptrs, void* clear_buf, int clear_rows, int* state, int rank,
                                          int world, const int* rows, const void* w, int T, int H, float eps,
                                          void* zero_ptr, long long zero_bytes, int flags, atx_stream_t stream);

/* Low-latency variant for decode-sized steps: no flag barrier and no pulls. Every buffer a peer writes into is
 * kept filled with a sentinel bit pattern (-0.0: fp32 0x80000000, bf16 0x8000; payloads are sanitised so they
 * never contain it) and the receiver spins on the data itself. Ownership of rows as above (t mod world).
 *   part        this rank's partial sums [T, H] fp32 (LOCAL memory; read only)
 *   rs_ptrs[p]  rank p's receive slots for THIS parity, fp32 [world][T_cap][H], peer-mapped, sentinel-filled once
 *               at start-up (the kernel re-arms what it reads)
 *   out_ptrs[p] rank p's activation buffer for THIS parity, bf16 [>= T, H], peer-mapped, sentinel in rows [0, T)
 *               when the call starts
 *   reset_ptr / reset_bytes  LOCAL region filled with the bf16 sentinel: the OTHER parity's activation rows,
 *               which the GEMMs before this call have finished reading (16-byte multiple)
 *   clear_buf / clear_rows, zero_ptr / zero_bytes, rows, x, w  as in the flag-barrier form (local housekeeping)
 * Calls must alternate between two parities (two rs / out buffer sets), every rank making the same calls in
 * the same order. The whole grid (T x ceil(H/2048) CTAs) spins on remote data and must be co-resident: rejected
 * otherwise. Latency per call, 1 MiB message: see profiles/ (ar_microbench). */
int atx_allreduce_add_rmsnorm_ll(float* x, const float* part, void* const* rs_ptrs, void* const* out_ptrs,
                                 void* clear_buf, int clear_rows, void* reset_ptr, long long reset_bytes, int T_cap,
                                 int rank, int world, const int* rows, const void* w, int T, int H, float eps,
                                 void* zero_ptr, long long zero_bytes, int flags, atx_stream_t stream);

/* ---- RoPE + KV-cache write ------------------------------------------------------------------------
 * Replaces apply_rotary_pos_emb (modeling_llama.py:146-168, rotate_half layout :138-143) and
 * past_key_values.update (:267) / vLLM reshape_and_cache. qkv: [T, (Hq + 2*Hkv) * D] fp32 (GEMM
 * output), cos_sin: [max_pos, D] fp32 (row p = cos(p*inv_freq[0..D/2)) ++ sin(...)), positions[T],
 * slots[T] (slot = block * block_size + offset; negative = skip the cache write).
 * q_out: [T, Hq * D] bf16. K and V caches: [num_blocks, Hkv, block_size, D] bf16 each. */
int atx_rope_kv_write(const float* qkv, const int* positions, const int* slots, const float* cos_sin,
                      void* q_out, void* k_cache, void* v_cache, int T, int Hq, int Hkv, int D,
                      int block_size, int flags, atx_stream_t stream);

/* ---- SwiGLU: act[t, i] = bf16( silu(gu[t, i]) * gu[t, I + i] ) ------------------------------------
 * Replaces LlamaMLP.forward's act_fn(gate) * up (modeling_llama.py:182-184). gu: [T, 2*I] fp32. */
int atx_silu_mul(const float* gu, void* act, int T, int I, int flags, atx_stream_t stream);

/* ---- paged attention, decode (one query token per sequence) ---------------------------------------
 * Replaces eager_attention_forward (modeling_llama.py:199-222; repeat_kv :187-196; fp32 softmax
 * :217) over vLLM's paged KV (FlashInfer decode). q: [B, Hq * D] bf16; out: [B, Hq * D] bf16;
 * block_table: [B, max_blocks] int32; seq_lens[B] = tokens in cache INCLUDING the current one.
 * workspace: fp32 scratch of atx_paged_attn_decode_workspace_bytes(B, Hq, D, num_splits) bytes,
 * supplied by the caller (partial outputs + running max / sum per split).
 * head_dim 64 | 128, at most 8 query heads per KV head, block_size a multiple of 16 (else ATX_ERR_UNSUPPORTED). */
long long atx_paged_attn_decode_workspace_bytes(int B, int Hq, int D, int num_splits);
int atx_paged_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                          const int* seq_lens, void* out, void* workspace, long long workspace_bytes,
                          int B, int Hq, int Hkv, int D, int block_size, int max_blocks, int num_splits,
                          float scale, int flags, atx_stream_t stream);

/* Decode attention for callers that cannot allocate device memory. (No counterpart in the reference:
 * it exists for hosts of this library, not for parity.) Same arithmetic and arguments as
 * atx_paged_attn_decode, but the per-split partial results are kept in an 8 MiB array that is built
 * into the library (resident on every GPU that loads it, until the process exits) instead of in a
 * caller buffer — for processes that have already committed all of their HBM (e.g. to a KV pool),
 * run under a fixed memory reservation, must avoid cudaMalloc's device-wide synchronisation on the
 * request path, or bind this ABI from a language runtime with no CUDA allocator of its own.
 *   - Limit: atx_paged_attn_decode_workspace_bytes(B, Hq, D, num_splits) must not exceed
 *     atx_paged_attn_decode_static_capacity() (8 MiB); larger requests return ATX_ERR_LIMIT with the
 *     sizes spelled out in atx_last_error(). It never calls cudaMalloc / cudaFree.
 *   - The first call on each device looks up the array's device address (one host-side runtime
 *     query, with that device current); make that first call before starting any stream capture.
 *   - All calls on a device share the one array and it keeps whatever the last call left in it.
 *     Nothing needs clearing between calls (each call overwrites every slot it later reads), but two
 *     calls whose kernels overlap on the GPU — different streams, or different host threads — race
 *     on it: serialise them (same stream, or an event) or use the caller-scratch entry point. */
long long atx_paged_attn_decode_static_capacity(void);
int atx_paged_attn_decode_static(const void* q, const void* k_cache, const void* v_cache,
                                 const int* block_table, const int* seq_lens, void* out, int B, int Hq,
                                 int Hkv, int D, int block_size, int max_blocks, int num_splits, float scale,
                                 int flags, atx_stream_t stream);

/* ---- paged attention, prefill / chunked prefill (causal) ------------------------------------------
 * Same arithmetic as above with the causal mask of create_causal_mask; queries of sequence s are
 * rows [cu_q[s], cu_q[s+1]) of q, and their keys are the first ctx_lens[s] cache tokens of that
 * sequence (the chunk's own K/V must already be in the cache): query j of n attends to keys
 * [0, ctx_lens[s] - n + j]. q/out: [total_q, Hq * D] bf16 (total_q = cu_q[S]); num_blocks = blocks in
 * each cache (they bound the TMA descriptors). One kernel, on tcgen05: head_dim 64 | 128, block_size 16,
 * 16-byte aligned buffers; anything else returns ATX_ERR_UNSUPPORTED. */
int atx_paged_attn_prefill(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                           const int* cu_q, const int* ctx_lens, void* out, int S, int max_q_len,
                           long long total_q, long long num_blocks, int Hq, int Hkv, int D, int block_size,
                           int max_blocks, float scale, int flags, atx_stream_t stream);

/* ---- sampler --------------------------------------------------------------------------------------
 * Replaces vLLM SamplingParams(temperature=0.2) (llm/serve_llm.py:379, 521) / HF do_sample
 * (llm/hf_cpu_server.py:91) and greedy arg-max used for parity. logits: [B, ldl] fp32, V valid.
 * temperature[b] <= 0 => arg-max (lowest index wins ties, as torch.argmax). Otherwise an exact
 * categorical draw from softmax(logits / temperature) restricted to the top-p nucleus, by the
 * Gumbel-max rule with the counter-based generator documented in oracle/sampler_ref.py
 * (seeds[b], steps[b] select the stream). out_ids: [B] int32. */
int atx_sample(const float* logits, long long ldl, const float* temperature, const float* top_p,
               const unsigned long long* seeds, const int* steps, int* out_ids, int B, int V, int flags,
               atx_stream_t stream);

/* Vocabulary-parallel form of the above (tensor parallelism: each rank holds V / world columns of every logits row,
 * the LM head being sharded by vocabulary): atx_sample_shard reduces this rank's shard of each row to ONE
 * (score, global index) pair — the logit for greedy rows, logit / T + Gumbel noise keyed by the GLOBAL token index
 * otherwise — and atx_sample_merge, given the `world` shards' pairs ([world][B] float2: score, index bits), picks the
 * best (lowest index on ties): exactly the token atx_sample draws from the assembled row, with 8 bytes per row and
 * rank exchanged instead of the row itself. Replaces the logits all-gather vLLM performs before its sampler under
 * tensor parallelism (reached through llm/serve_llm.py:374-379). No top-p here (it needs the whole row's sum). */
int atx_sample_shard(const float* logits, long long ldl, int idx_offset, const float* temperature,
                     const unsigned long long* seeds, const int* steps, void* pairs, int B, int V_local, int flags,
                     atx_stream_t stream);
int atx_sample_merge(const void* pairs, int world, int B, int* out_ids, int flags, atx_stream_t stream);

/* ---- Element type of weights, GEMM-input activations and KV pages in the calls below ------------------------------ */
#define ATX_DT_BF16 0
#define ATX_DT_F32 1

/* out[t, n] (+)= sum_k X[t, k] * W[n, k] on the FMA pipe: fp32 operands (true 32-bit products), or shapes the tcgen05
 * plan refuses (K not a multiple of 64). Any N, K, T and row pitches; fp32 accumulation in a fixed order. */
int atx_gemm_simple(const void* W, long long ldw, const void* X, long long ldx, float* out, long long ldo, int T, int N,
                    int K, int add, int dtype, int flags, atx_stream_t stream);

/* ---- Mixers with a recurrent state, and what surrounds them ---------------------------------------------------------
 * A step is a flat batch of rows. Sequence s owns rows [seq_start[s], seq_start[s] + seq_count[s]); its first row is
 * position seq_pos0[s]; tok_seq[t] is the sequence of row t (-1: padded row); seq_slot[s] is the state slot. A sequence
 * at position 0 starts from zero state whatever the slot held before. seq_count 0 marks a padded entry. */

/* out[t, :] = table[ids[t], :] as fp32, any width. */
int atx_embed_rows(const int* ids, const void* table, float* out, int T, int W, int V, int dtype, int flags,
                   atx_stream_t stream);
/* out[t, :] = [ h[t, :] rounded to the element type ; table[ids[t], :] ]  (2 W columns). */
int atx_concat_embed(const float* h, const int* ids, const void* table, void* out, int T, int W, int V, int dtype,
                     int flags, atx_stream_t stream);
/* Residual update between two RMS norms, one pass over the row:
 *   h[r] += rms(y[r]) * w_post  (if y)  + vec (if vec);   out[t] = rms(h[r]) * w_pre  (if w_pre);   r = rows ? rows[t] : t
 * rms(x) = x / sqrt(mean(x^2) + eps). With `rows` the residual is read only. zero_y != 0 clears each row of y once it
 * has been read, and spare CTAs clear zero_ptr / zero_bytes (a multiple of 16): the accumulators of the split-K GEMMs
 * that run next. */
int atx_resid_norm(float* h, float* y, const void* w_post, const void* vec, const void* w_pre, void* out,
                   const int* rows, int T, int W, float eps, int zero_y, void* zero_ptr, long long zero_bytes, int dtype,
                   int flags, atx_stream_t stream);
/* out[t, i] = silu(gu[t, i]) * gu[t, I + i] */
int atx_gated_act(const float* gu, void* out, int T, int I, int dtype, int flags, atx_stream_t stream);
/* Gated RMS norm over n / groups consecutive elements at a time:
 *   mode 0: out = rms(y) * w * sigmoid(gate) * scale;   mode 1: out = rms(y * silu(gate)) * w * scale */
int atx_gated_norm(const float* y, long long ldy, const float* gate, long long ldg, const void* w, void* out,
                   long long ldo, int T, int n, int groups, float eps, int mode, float scale, int dtype, int flags,
                   atx_stream_t stream);
/* Short causal convolution over C channels (taps K, last tap = the row itself) + bias + silu, with the raw inputs of the
 * K - 1 positions before the step taken from conv_state [slots, K - 1, C]; and per head dt = softplus(in[dt_off + h] +
 * dt_bias[h]), decay = exp(-exp(a_log[h]) * dt). xbc [T, C], dt_out / decay_out [T, H], all fp32. */
int atx_conv_dt(const float* in, long long ld, int x_off, int dt_off, const void* w, const void* b, const void* dt_bias,
                const void* a_log, const float* conv_state, float* xbc, float* dt_out, float* decay_out,
                const int* tok_seq, const int* seq_start, const int* seq_pos0, const int* seq_slot, int T, int C, int H,
                int K, int dtype, int flags, atx_stream_t stream);
/* conv_state <- raw inputs of each sequence's last K - 1 positions (run after atx_conv_dt of the same step). */
int atx_conv_state_update(const float* in, long long ld, int x_off, float* conv_state, const int* seq_start,
                          const int* seq_count, const int* seq_pos0, const int* seq_slot, int n_seqs, int C, int K,
                          int flags, atx_stream_t stream);
/* Decayed outer-product recurrence per head, state fp32 [slots, H, D, V]:
 *   S_t = a_t S_(t-1) + (c_t k_t) v_t^T,   y_t = S_t^T q_t + d v_t
 * a_t = decay_head[h] or decay_tok[t, h]; c_t = kscale_tok[t, h] or 1; d = skip[h] or 0; q/k of head h come from group
 * h / (H / G) at columns [group * D, ...), v and y from columns [h * V, ...); act = 1: silu on q, k, v as read. */
int atx_linear_recurrence(const float* q, long long ldq, const float* k, long long ldk, const float* v, long long ldv,
                          int H, int G, int D, int V, const float* decay_head, const float* decay_tok,
                          const float* kscale_tok, const float* skip, int act, float* state, float* y, long long ldy,
                          const int* seq_start, const int* seq_count, const int* seq_pos0, const int* seq_slot,
                          int n_seqs, int flags, atx_stream_t stream);
/* The same recurrence for prompt portions in its chunk-parallel form on the tensor cores (chunks of 64 tokens: the
 * products inside a chunk and with the state before it are bf16 MMAs with fp32 accumulation; state, logarithms of the
 * decays, their running sums, exponentials and step sizes stay fp32). Same arguments, same state layout, so a sequence
 * may switch between the two from step to step. D must be one of the sizes ..._supported() accepts. */
int atx_linear_recurrence_chunked_supported(int D);
int atx_linear_recurrence_chunked(const float* q, long long ldq, const float* k, long long ldk, const float* v,
                                  long long ldv, int H, int G, int D, int V, const float* decay_head,
                                  const float* decay_tok, const float* kscale_tok, const float* skip, int act,
                                  float* state, float* y, long long ldy, const int* seq_start, const int* seq_count,
                                  const int* seq_pos0, const int* seq_slot, int n_seqs, int flags, atx_stream_t stream);
/* q/k/v of one step from a fused projection (fp32, row pitch ld, column offsets): + bias (nullable), RMS norm over the
 * WHOLE q and the whole k projection with weights wq [H D] / wk [G D] (nullable: no norm), rotation of adjacent pairs
 * (2i, 2i+1) of the first rot_dims dimensions of every head by the angles of table rot [max_pos, rot_dims] (cosines,
 * then sines), q -> q_out [T, H D], k / v -> pages K [blocks, G, bs, D], V [blocks, G, bs, Vd] at slots[t]. */
int atx_qk_prepare(const float* proj, long long ld, int q_off, int k_off, int v_off, const void* bq, const void* bk,
                   const void* bv, const void* wq, const void* wk, const float* rot, int rot_dims, const int* positions,
                   const int* slots, void* q_out, void* k_cache, void* v_cache, int T, int H, int G, int D, int Vd,
                   int block_size, float eps, int dtype, int flags, atx_stream_t stream);
/* Attention of every row over its sequence's pages: score = (q . k) * scale, capped as softcap * tanh(score / softcap)
 * if softcap > 0; a query at position p sees keys j <= p with floor(j / chunk) == floor(p / chunk) (chunk 0: all j <= p);
 * sink != 0 adds 1 to the softmax denominator; out = softmax . V * sigmoid(gate[t, h]) (gate nullable) * out_scale. */
int atx_attn_local(const void* q, const void* k_cache, const void* v_cache, const int* block_tables, int max_blocks,
                   const int* tok_seq, const int* positions, const float* gate, long long ldg, void* out, long long ldo,
                   int T, int H, int G, int D, int Vd, int block_size, float scale, float softcap, int chunk, int sink,
                   float out_scale, int dtype, int flags, atx_stream_t stream);
/* The same attention for prompt portions on the tensor cores (mma.sync m16n8k16, bf16 operands, fp32 softmax and
 * accumulation): sequences are given as (first row, rows, first position) triples, block_tables has one row per listed
 * sequence. ..._supported() says whether the head sizes and element type have a tensor-core kernel (else use
 * atx_attn_local for those rows too). total_rows bounds the sum of the sequences' rows. */
int atx_attn_local_prefill_supported(int D, int Vd, int dtype);
int atx_attn_local_prefill(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                           int max_blocks, const int* seq_start, const int* seq_count, const int* seq_pos0, int n_seqs,
                           int total_rows, const float* gate, long long ldg, void* out, long long ldo, int H, int G, int D,
                           int Vd, int block_size, float scale, float softcap, int chunk, int sink, float out_scale,
                           int dtype, int flags, atx_stream_t stream);

/* ---- Attention variants and per-head operations that further designs are built from ---------------------------------
 * (Gopopel: sliding-window attention with a distance penalty and a learned sink, latent attention in its absorbed
 * form, tanh norm, squared-ReLU feed-forward. Every constant is an argument.) */

/* out[t, :] = table[ids[t], :] * scale as fp32. */
int atx_embed_rows_scaled(const int* ids, const void* table, float* out, int T, int W, int V, float scale, int dtype,
                          int flags, atx_stream_t stream);
/* out[t, :] = tanh(alpha * x[r, :]) * w + b, r = rows ? rows[t] : t: a norm without row statistics. x fp32 [., W], w / b /
 * out of the element type. Spare CTAs clear zero_ptr / zero_bytes (a multiple of 16): the accumulator of a split-K GEMM
 * that runs next. */
int atx_tanh_norm(const float* x, const int* rows, float alpha, const void* w, const void* b, void* out, int T, int W,
                  void* zero_ptr, long long zero_bytes, int dtype, int flags, atx_stream_t stream);
#define ATX_ACT_RELU2 0     /* max(z, 0)^2 */
#define ATX_ACT_GELU_TANH 1 /* z/2 (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))) */
/* out[t, i] = act(in[t, i]) (fp32 in, element type out). */
int atx_unary_act(const float* in, long long ldi, void* out, long long ldo, int T, int I, int kind, int dtype, int flags,
                  atx_stream_t stream);

/* One slice of a fused projection row, cut into `heads` heads of `width` elements (head h starts at column
 * src_off + h * src_stride). Per head, in this order: the first norm_dims elements are divided by their root mean square
 * (eps under the root) and multiplied by norm_w; the elements [rot_off, rot_off + rot_dims) are rotated in adjacent pairs
 * (or, with rot_half, in pairs half the range apart) by the angles of rot [max_pos, rot_dims] (cosines, then sines) at
 * the row's position; `save` (fp32 [T, heads * width])
 * receives the result; with mix_src (same shape) the result becomes (1 - mix) * result + mix * mix_src. It is written as
 * the element type to rows (dst [T, dst_ld], head h at column dst_off + h * dst_stride) or to pages
 * (dst [blocks, heads, block_size, dst_stride], at the row's slot, from column dst_off of the token's row). */
#define ATX_HEAD_DST_ROWS 0
#define ATX_HEAD_DST_PAGES 1
#define ATX_HEAD_SEGS_MAX 4
typedef struct atx_head_seg {
    int src_off, src_stride, heads, width;
    int norm_dims, rot_off, rot_dims;
    int dst_kind, dst_off, dst_stride;
    float mix;
    int rot_half; /* 0: adjacent pairs (2i, 2i+1); 1: element i pairs with i + rot_dims/2, angle i of the table */
    const void* norm_w;
    const float* rot;
    const float* mix_src;
    float* save;
    void* dst;
    long long dst_ld;
} atx_head_seg;
int atx_head_prepare(const float* src, long long ld, const atx_head_seg* segs, int n_segs, const int* positions,
                     const int* slots, int T, int block_size, float eps, int dtype, int flags, atx_stream_t stream);
/* A small matrix product per head: out[t, o_off + h * o_head_stride + n] = sum_k X[t, x_off + h * x_head_stride + k] *
 * W[(h * N + n) * ldw + k], times sigmoid(gate[t, h * N + n]) if gate. X fp32 (x_f32 != 0) or of the element type, gate
 * fp32, W and out of the element type. bf16 runs on the tensor cores (X rounded to bf16, fp32 accumulation) unless
 * ATX_FLAG_HEAD_GEMM_FMA asks for the FMA pipe (X as given, bf16 weights widened exactly); fp32 always takes the FMA pipe. */
#define ATX_FLAG_HEAD_GEMM_FMA 8
int atx_head_gemm(const void* X, int x_f32, long long ldx, int x_off, int x_head_stride, const void* W, long long ldw,
                  const float* gate, long long ldg, void* out, long long ldo, int o_off, int o_head_stride, int T,
                  int heads, int N, int K, int dtype, int flags, atx_stream_t stream);

/* atx_attn_local with the remaining options of the kernel: a token's key row holds k_row elements (the first D are the
 * key) and its value row v_row (the first Vd are the value), so that keys and values may live in one page array (latent
 * attention: v_cache = k_cache, Vd leading elements); window > 0: a query at p sees only keys j > p - window (on top of
 * j <= p and of `chunk`); slopes [H] (nullable): slopes[h] * (p - j) is taken off the score after scale and cap;
 * sinks [H] (nullable): exp(sinks[h]) is added to the softmax denominator (sink != 0 without sinks: exp(0)). */
int atx_attn_window(const void* q, const void* k_cache, const void* v_cache, long long k_row, long long v_row,
                    const int* block_tables, int max_blocks, const int* tok_seq, const int* positions, const float* gate,
                    long long ldg, void* out, long long ldo, int T, int H, int G, int D, int Vd, int block_size,
                    float scale, float softcap, int chunk, int window, const float* slopes, const float* sinks, int sink,
                    float out_scale, int dtype, int flags, atx_stream_t stream);
/* atx_attn_window for prompt portions on the tensor cores (the kernel of atx_attn_local_prefill with the same further
 * options): bf16, key size up to 256 and value size up to 128, head and row sizes in multiples of 8 elements; sizes
 * between the kernel's tile widths run on the next wider tile with zero columns. ..._supported() says whether a shape has
 * this kernel (else use atx_attn_window for those rows too). */
int atx_attn_window_prefill_supported(int D, int Vd, long long k_row, long long v_row, int dtype);
int atx_attn_window_prefill(const void* q, const void* k_cache, const void* v_cache, long long k_row, long long v_row,
                            const int* block_tables, int max_blocks, const int* seq_start, const int* seq_count,
                            const int* seq_pos0, int n_seqs, int total_rows, const float* gate, long long ldg, void* out,
                            long long ldo, int H, int G, int D, int Vd, int block_size, float scale, float softcap,
                            int chunk, int window, const float* slopes, const float* sinks, int sink, float out_scale,
                            int dtype, int flags, atx_stream_t stream);
/* atx_attn_window for single decoded tokens on the tensor cores: one CTA per (token, key/value head, slice of the keys),
 * the query heads that share the key/value head being the rows of its tile (at most 64 of them), so keys and values are
 * read once per group; `splits` slices leave partial results in `workspace` (..._workspace_bytes(), 8-byte aligned;
 * none for one slice) and a second kernel folds them. Same shapes as atx_attn_window_prefill. */
int atx_attn_window_decode_supported(int H, int G, int D, int Vd, long long k_row, long long v_row, int dtype);
long long atx_attn_window_decode_workspace_bytes(int T, int H, int Vd, int splits);
int atx_attn_window_decode(const void* q, const void* k_cache, const void* v_cache, long long k_row, long long v_row,
                           const int* block_tables, int max_blocks, const int* tok_seq, const int* positions,
                           const float* gate, long long ldg, void* out, long long ldo, void* workspace,
                           long long workspace_bytes, int splits, int T, int H, int G, int D, int Vd, int block_size,
                           float scale, float softcap, int chunk, int window, const float* slopes, const float* sinks,
                           int sink, float out_scale, int dtype, int flags, atx_stream_t stream);

/* ---- Further mechanisms: a residual branch scale, rows that read their predecessor, attention without a softmax,
 * a polynomial activation of unit-rms powers, a mixture of experts. (Zonidra is built from these; every constant is an
 * argument.) */

/* atx_resid_norm with a second weight vector on the post-normed sublayer output, h[r] += rms(y[r]) * w_post * post_scale
 * (post_scale nullable), and with `out` as fp32 when out_f32 != 0 (else the element type). */
int atx_resid_norm_scaled(float* h, float* y, const void* w_post, const void* post_scale, const void* vec,
                          const void* w_pre, void* out, int out_f32, const int* rows, int T, int W, float eps, int zero_y,
                          void* zero_ptr, long long zero_bytes, int dtype, int flags, atx_stream_t stream);
/* out[t, :] = table[ids[t], :] * scale + pair_table[r, :] with r = (ids[t-1] * mul_prev + ids[t] * mul_cur) mod buckets, or
 * r = buckets (the table's last row) for the first token of a sequence. The predecessor of a step's first row is
 * prev_tok[seq_slot[s]], which then receives the step's last token of the sequence. Rows with tok_seq < 0 become zeros. */
int atx_embed_rows_pair(const int* ids, const void* table, float scale, const void* pair_table, int buckets, int mul_prev,
                        int mul_cur, int* prev_tok, const int* tok_seq, const int* seq_start, const int* seq_count,
                        const int* seq_pos0, const int* seq_slot, float* out, int T, int W, int V, int dtype, int flags,
                        atx_stream_t stream);
/* out[t, :] = x[t, :] + (x[t-1, :] - x[t, :]) * mu (element type out, x fp32); x[-1] of a sequence is zero, the
 * predecessor of a step's first row is state[seq_slot[s], :] (fp32 [slots, W]), which then receives the step's last row. */
int atx_token_shift(const float* x, const void* mu, float* state, const int* tok_seq, const int* seq_start,
                    const int* seq_count, const int* seq_pos0, const int* seq_slot, void* out, int T, int W, int dtype,
                    int flags, atx_stream_t stream);
/* out[t, i] = a z / rms(z) + b z^2 / rms(z^2) + c z^3 / rms(z^3) + e, z = z[t, i], each rms over the row's F elements
 * (eps under the root); coef = {a, b, c, e} fp32 on the device. */
int atx_poly_norm_act(const float* z, long long ldz, const float* coef, void* out, long long ldo, int T, int F, float eps,
                      int dtype, int flags, atx_stream_t stream);

/* Options of the paged attention kernels (atx_attn_window* take the soft-max subset of them as plain arguments).
 * A query at position p sees key j when j <= p, floor(j / chunk) == floor(p / chunk) (chunk > 0), and j > p - window
 * (window > 0) or j < keep_first. score = cap(scale q.k) - slopes[h] (p - j) + bias[h]. weight SOFTMAX: soft-max over the
 * visible keys, `sink` / `sinks` adding exp(0) / exp(sinks[h]) to the denominator; SIGMOID: each visible key weighs
 * sigmoid(score), nothing is normalised (no sink). gate [T, H], or [T, H * Vd] with gate_elem: out *= sigmoid(gate). */
#define ATX_ATTN_SOFTMAX 0
#define ATX_ATTN_SIGMOID 1
typedef struct atx_attn_opts {
    float scale, softcap, out_scale;
    int chunk, window, keep_first, sink;
    int weight, gate_elem;
    const float* slopes;
    const float* sinks;
    const float* bias;
} atx_attn_opts;
/* The three attention entry points with every option: rows one by one (any element type), prompt portions on the tensor
 * cores, single decoded tokens on the tensor cores (see atx_attn_window, _prefill, _decode for shapes and limits). */
int atx_attn_paged(const void* q, const void* k_cache, const void* v_cache, long long k_row, long long v_row,
                   const int* block_tables, int max_blocks, const int* tok_seq, const int* positions, const float* gate,
                   long long ldg, void* out, long long ldo, int T, int H, int G, int D, int Vd, int block_size,
                   const atx_attn_opts* opts, int dtype, int flags, atx_stream_t stream);
int atx_attn_paged_prefill(const void* q, const void* k_cache, const void* v_cache, long long k_row, long long v_row,
                           const int* block_tables, int max_blocks, const int* seq_start, const int* seq_count,
                           const int* seq_pos0, int n_seqs, int total_rows, const float* gate, long long ldg, void* out,
                           long long ldo, int H, int G, int D, int Vd, int block_size, const atx_attn_opts* opts, int dtype,
                           int flags, atx_stream_t stream);
int atx_attn_paged_decode(const void* q, const void* k_cache, const void* v_cache, long long k_row, long long v_row,
                          const int* block_tables, int max_blocks, const int* tok_seq, const int* positions,
                          const float* gate, long long ldg, void* out, long long ldo, void* workspace,
                          long long workspace_bytes, int splits, int T, int H, int G, int D, int Vd, int block_size,
                          const atx_attn_opts* opts, int dtype, int flags, atx_stream_t stream);

/* Mixture of experts. logits [T, ld] fp32 hold R router outputs per token: soft-max over all R; the `top` largest of
 * score + correction[r] (correction nullable; lowest index on ties) are chosen: sel [T, top] int32, wgt [T, top] = score *
 * scale. At most 512 outputs. */
int atx_moe_route(const float* logits, long long ld, const float* correction, int R, int top, float scale, int* sel,
                  float* wgt, int T, int flags, atx_stream_t stream);
/* Sorts the n_pairs = T * top (token, choice) pairs by expert. Choices >= E (or < 0) take no slot. seg_off [E + 1]: first
 * slot of every expert; perm [n_pairs]: pair of a slot; slot_of [n_pairs]: slot of a pair (-1: none); tiles
 * [2 + 2 * max_tiles] int32: the tile count, a spare word, then (expert, first slot) per tile of tile_rows slots
 * (atx_moe_tile_rows() for atx_moe_expert_gemm, atx_gemm_grouped_tile_rows() for atx_gemm_run_grouped);
 * max_tiles = ceil(n_pairs / tile_rows) + E always suffices. */
int atx_moe_tile_rows(void);
int atx_moe_plan(const int* sel, int n_pairs, int E, int tile_rows, int* seg_off, int* perm, int* slot_of, int* tiles,
                 int flags, atx_stream_t stream);
/* out[slot, :] = x[perm[slot] / top, :] for the slots the plan handed out (at most max_slots): every expert's rows back to
 * back, for atx_gemm_run_grouped. */
int atx_moe_gather_rows(const void* x, long long ldx, const int* perm, int top, const int* seg_off, int E, void* out,
                        long long ldo, int max_slots, int W, int dtype, int flags, atx_stream_t stream);
/* out[slot, n] = sum_k A[row(slot), k] * W[e * expert_stride + n * ldw + k] for the slots of every expert e; row(slot) =
 * perm[slot] / top with gather != 0, else slot. gated == 0: fp32 out. gated != 0: W holds N gate rows then N up rows per
 * expert (interleaved != 0: blocks of 64 gate rows and 64 up rows in turn, the layout ATX_GEMM_SWIGLU_BF16 reads) and
 * out (element type) = silu(gate) * up. bf16 on the tensor cores, fp32 on the FMA pipe. tile_rows: the slots per tile the
 * plan was made with, atx_moe_tile_rows(), or 16 (bf16 only: decode-sized steps, more CTAs per SM). The grid covers
 * max_tiles tiles; CTAs beyond the plan's count return. */
int atx_moe_expert_gemm(const void* A, long long lda, const int* perm, int top, int gather, const void* W,
                        long long expert_stride, long long ldw, void* out, long long ldo, int N, int K, int gated,
                        int interleaved, int tile_rows, const int* seg_off, const int* tiles, int max_tiles, int dtype,
                        int flags, atx_stream_t stream);
/* y[t, :] = sigmoid(shared_gate[t * ldsg]) * y[t, :] (shared_gate nullable: y is overwritten) + sum_k wgt[t, k] *
 * (sel[t, k] >= E ? x[t, :] : ye[slot_of[t * top + k], :]). y, ye fp32; x of the element type. */
int atx_moe_combine(float* y, const float* ye, long long lde, const void* x, const int* sel, const float* wgt,
                    const int* slot_of, const float* shared_gate, long long ldsg, int T, int W, int top, int E, int dtype,
                    int flags, atx_stream_t stream);

/* ---- Further mechanisms: a norm behind a sublayer only, a residual short convolution in front of a mixer, a recurrence
 * whose state decays per key channel, clamped gates, renormalised expert weights. (Napuzen is built from these; every
 * constant is an argument.) */

/* atx_resid_norm_scaled where the consumer may read the stream without a norm: w_pre == NULL with out != NULL writes
 * out[t] = h[r] * out_scale (element type, or fp32 with out_f32); with w_pre, out[t] = rms(h[r]) * w_pre * out_scale. */
int atx_resid_norm_out(float* h, float* y, const void* w_post, const void* post_scale, const void* vec, const void* w_pre,
                       void* out, int out_f32, float out_scale, const int* rows, int T, int W, float eps, int zero_y,
                       void* zero_ptr, long long zero_bytes, int dtype, int flags, atx_stream_t stream);
/* out[t, i] = g * sigmoid(alpha * g) * (u + shift), g = min(gu[t, i], limit), u = clamp(gu[t, I + i], -limit, limit). */
int atx_gated_act_clamped(const float* gu, void* out, int T, int I, float alpha, float limit, float shift, int dtype,
                          int flags, atx_stream_t stream);
/* atx_gated_norm with mode 2: out = rms(y) * w * silu(gate) * scale, and with w_shared != 0: w holds n / groups weights
 * that every group uses (a norm per head with one weight vector for all heads). */
int atx_gated_norm_groups(const float* y, long long ldy, const float* gate, long long ldg, const void* w, int w_shared,
                          void* out, long long ldo, int T, int n, int groups, float eps, int mode, float scale, int dtype,
                          int flags, atx_stream_t stream);
/* out[t, c] = x[t, c] + sum_j w[c, j] * x[t - (K - 1 - j), c] over the rows of t's sequence (K taps; w [C, K] of
 * the element type; no bias, no activation): x fp32 [T, ld], out of the element type [T, ldo]. The K - 1 rows before a
 * step come from conv_state [slots, K - 1, C] fp32, which atx_conv_state_update(x, ld, 0, ...) refreshes after this call;
 * rows before position 0 are zero. Rows with tok_seq < 0 are skipped. */
int atx_conv_residual(const float* x, long long ld, const void* w, const float* conv_state, void* out, long long ldo,
                      const int* tok_seq, const int* seq_start, const int* seq_pos0, const int* seq_slot, int T, int C,
                      int K, int dtype, int flags, atx_stream_t stream);
/* out[t, c] = log(sigmoid(b[c] + sum_r A[c, r] * lo[t, r])) / tau, fp32: the logarithm of a decay factor in (0, 1) per
 * channel from a narrow projection lo [T, ld] fp32 (R columns); A [C, R], b [C] (nullable) of the element type. */
int atx_lowrank_logdecay(const float* lo, long long ld, const void* A, const void* b, float* out, long long ldo, int T,
                         int C, int R, float tau, int dtype, int flags, atx_stream_t stream);
/* atx_linear_recurrence with a decay per key channel: S_t = diag(a_t) S_(t-1) + k_t v_t^T, y_t = S_t^T (qscale q_t), with
 * a_t[d] = exp(ldecay[t, h * D + d]) (pitch ldc). State fp32 [slots, H, D, V]; q, k [., H * D], v, y [., H * V] fp32. */
int atx_gated_linear_recurrence(const float* q, long long ldq, const float* k, long long ldk, const float* v, long long ldv,
                                const float* ldecay, long long ldc, int H, int D, int V, float qscale, float* state,
                                float* y, long long ldy, const int* seq_start, const int* seq_count, const int* seq_pos0,
                                const int* seq_slot, int n_seqs, int flags, atx_stream_t stream);
/* The same recurrence for prompt portions in a chunk-parallel form on the tensor cores (chunks of 16 tokens: state read-out,
 * pair weights times values and the state update are bf16 MMAs with fp32 accumulation; the pair weights inside a chunk, the
 * state, the logarithms, their running sums and every exponential stay fp32). Same arguments and state layout, so a
 * sequence may switch between the two from step to step. D must be one of the sizes ..._supported() accepts. */
int atx_gated_linear_recurrence_chunked_supported(int D);
int atx_gated_linear_recurrence_chunked(const float* q, long long ldq, const float* k, long long ldk, const float* v,
                                        long long ldv, const float* ldecay, long long ldc, int H, int D, int V, float qscale,
                                        float* state, float* y, long long ldy, const int* seq_start, const int* seq_count,
                                        const int* seq_pos0, const int* seq_slot, int n_seqs, int flags,
                                        atx_stream_t stream);
/* atx_moe_route with normalize != 0: wgt = score / (sum of the chosen scores + 1e-20) * scale. */
int atx_moe_route_opts(const float* logits, long long ld, const float* correction, int R, int top, float scale,
                       int normalize, int* sel, float* wgt, int T, int flags, atx_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* ATX_B200_H */
