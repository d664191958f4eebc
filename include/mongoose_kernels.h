/*
 * libmongoose_kernels.so for NVIDIA B200 (sm_100a): C ABI.
 *
 * Two groups of entry points live in the one shared library:
 *
 *  1. mongoose_*  - the symbols mongoose's Go side resolves with dlsym
 *     (kernels.go:150-226, cuda_graph.go:226-234).  Signatures, argument
 *     meaning and the void/no-status convention are the reference's: every
 *     pointer is a caller-owned device address, work is enqueued on the
 *     given stream, nothing is allocated or freed.
 *
 *  2. mg_*  - a handle-based decode engine that mirrors CUDAFusedInference
 *     (cuda_fused_infer.go:75-142): create with the model dims, set weights
 *     with the reference's slot index scheme, step one token.  Calls return
 *     an int status (0 = ok) and never abort.
 *
 * No torch, no C++ types: plain pointers and sizes only.
 */
#ifndef MONGOOSE_KERNELS_H
#define MONGOOSE_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef __DRIVER_TYPES_H__
typedef struct CUstream_st* cudaStream_t;
#endif

/* Exported from the shared library (everything else is built with hidden visibility). */
#if defined(__GNUC__)
#define MG_API __attribute__((visibility("default")))
#else
#define MG_API
#endif

/* ------------------------------------------------------------------ */
/* 1. Reference ABI                                                    */
/* ------------------------------------------------------------------ */

/* In-place RMSNorm of x[seqLen, dim] with eps 1e-6.
 * Replaces kernels/mongoose.cu:16-56 (fn_rmsnorm, kernels.go:13).  Mandatory symbol. */
MG_API void mongoose_rmsnorm(float* x, const float* weight, int seqLen, int dim, cudaStream_t stream);
/* out = rmsnorm(in) * weight.  Replaces mongoose.cu:145-179 (fn_rmsnorm_out, kernels.go:14). */
MG_API void mongoose_rmsnorm_out(const float* in, float* out, const float* weight, int seqLen, int dim,
                          cudaStream_t stream);
/* out = rmsnorm(a + b) * weight.  Replaces mongoose.cu:370-410 (fn_fused_add_rmsnorm, kernels.go:21). */
MG_API void mongoose_fused_add_rmsnorm(const float* a, const float* b, float* out, const float* weight, int seqLen,
                                int dim, cudaStream_t stream);
/* x = max(x, 0).  Replaces mongoose.cu:192-199 (fn_relu, kernels.go:15).  Mandatory symbol. */
MG_API void mongoose_relu(float* x, int n, cudaStream_t stream);
/* a += b.  Replaces mongoose.cu:211-219 (fn_add_inplace, kernels.go:18).  Mandatory symbol. */
MG_API void mongoose_add_inplace(float* a, const float* b, int n, cudaStream_t stream);
/* out[i] = tokEmb[tokens[i]] + posEmb[i].  Replaces mongoose.cu:232-246
 * (fn_embedding_gather, kernels.go:20).  Mandatory symbol. */
MG_API void mongoose_embedding_gather(float* out, const float* tokEmb, const float* posEmb, const int* tokens,
                               int seqLen, int dim, cudaStream_t stream);
/* out[i] = embed[tokens[i]].  Replaces mongoose.cu:1050-1064 (fn_embed_gather2, kernels.go:35). */
MG_API void mongoose_embed_gather(float* out, const float* embed, const int* tokens, int seqLen, int dim,
                           cudaStream_t stream);
/* out = gate * sigmoid(gate) * up.  Replaces mongoose.cu:947-960 (fn_silu_gate_mul, kernels.go:30). */
MG_API void mongoose_silu_gate_mul(const float* gate, const float* up, float* out, int n, cudaStream_t stream);
/* Rotate-half RoPE in place on x[seqLen, dim]; tables indexed [pos*half + j].
 * Replaces mongoose.cu:987-1013 (fn_rope, kernels.go:32). */
MG_API void mongoose_rope(float* x, const float* cosTab, const float* sinTab, int seqLen, int dim, int headDim,
                   int nHeads, cudaStream_t stream);
/* cache[pos*kvDim + i] = src[i] (fp32).  Replaces mongoose.cu:1643-1653 (fn_kv_cache_write, kernels.go:61). */
MG_API void mongoose_kv_cache_write(float* cache, const float* src, int pos, int kvDim, cudaStream_t stream);
/* One query position against an fp32 KV cache [cacheLen, kvDim], grouped-query heads.
 * Replaces mongoose.cu:853-945 (fn_decode_attn, kernels.go:37). */
MG_API void mongoose_decode_attention(const float* Q, const float* Kcache, const float* Vcache, float* out,
                               int cacheLen, int dim, int kvDim, int nHeads, int nKVHeads,
                               cudaStream_t stream);
/* Per-row INT8 matvec: out[r] = sum_k act[k] * w[r,k] * (scales[r]/127).
 * Replaces mongoose.cu:1554-1595 (fn_q8_matvec, kernels.go:59). */
MG_API void mongoose_q8_matvec(const float* act, const void* w_i8, const float* scales, float* out, int N, int K,
                        cudaStream_t stream);
/* Per-row 4-bit matvec: byte k = elements 2k (low) and 2k+1 (high), value (nib-8)*scales[r]/7.
 * Replaces mongoose.cu:1597-1641 (fn_q4_matvec, kernels.go:60). */
MG_API void mongoose_q4_matvec(const float* act, const void* w_packed, const float* scales, float* out, int N,
                        int K, cudaStream_t stream);
/* GGUF Q4_0 matvec on raw 18-byte blocks (fp16 d + 16 nibble bytes; byte j = element j low,
 * element j+16 high; value d*(nib-8)), fp32 activations.
 * Declared at kernels.go:62 (fn_q4_0_matvec), resolved at kernels.go:206; the reference ships no source. */
MG_API void mongoose_q4_0_matvec(const float* act, const void* w_blocks, float* out, int N, int K,
                          cudaStream_t stream);
/* Activation -> int8 blocks of 32: 40 bytes each {float d; float sum; int8 q[32]} with d = amax/127,
 * sum = d * sum(q).  Declared at kernels.go:64 (fn_q8_quantize_act); scratch sizing (K/32)*40 at
 * cuda_fused_infer.go:173-176. */
MG_API void mongoose_q8_quantize_act(const float* act, void* q8_out, int K, cudaStream_t stream);
/* B activation vectors [B, K] -> [B, K/32] blocks.  Declared at kernels.go:67. */
MG_API void mongoose_q8_quantize_act_batch(const float* acts, void* q8_out, int K, int B, cudaStream_t stream);
/* Q4_0 matvec with integer dot products: quantizes act into `scratch` ((K/32)*40 bytes, caller-owned),
 * then int4 x int8 dp4a.  Declared at kernels.go:63 (fn_q4_0_matvec_dp4a). */
MG_API void mongoose_q4_0_matvec_dp4a(const float* act, const void* w_blocks, float* out, int N, int K,
                               void* scratch, cudaStream_t stream);
/* Same with a pre-quantized activation.  Declared at kernels.go:65. */
MG_API void mongoose_q4_0_matvec_dp4a_preq(const void* w_blocks, const void* q8, float* out, int N, int K,
                                    cudaStream_t stream);
/* B pre-quantized activations; out is [B, N].  Declared at kernels.go:66. */
MG_API void mongoose_q4_0_matvec_dp4a_batch(const void* w_blocks, const void* q8, float* out, int N, int K, int B,
                                     cudaStream_t stream);
/* Q4_0 integer-dot matvec for callers that cannot allocate device memory (allocator calls forbidden
 * in the section they run in, or no budget left to carve a scratch buffer from): the activation
 * blocks live in a fixed 40 KiB array inside the library instead of a caller buffer, so K is limited
 * to 32768.  No counterpart in the reference.  The first call on each device resolves the array's
 * device address (make it before any stream capture); calls share the array, so calls that overlap
 * on the GPU race.  Returns MG_OK / MG_ERR_ARG / MG_ERR_CUDA. */
MG_API int mongoose_q4_0_matvec_dp4a_static(const float* act, const void* w_blocks, float* out, int N, int K,
                                            cudaStream_t stream);
/* Text of the last error mongoose_q4_0_matvec_dp4a_static returned on the calling thread ("" if none). */
MG_API const char* mongoose_static_scratch_error(void);
/* Replaces mongoose.cu:355-368 (fn_copy / fn_zero / fn_sync, kernels.go:24-26). */
MG_API void mongoose_copy(void* dst, const void* src, size_t bytes, cudaStream_t stream);
MG_API void mongoose_zero(void* ptr, size_t bytes, cudaStream_t stream);
MG_API void mongoose_sync(cudaStream_t stream);
/* Replaces mongoose.cu:1415-1438 (fn_fp32_to_fp16 / fn_fp16_to_fp32, kernels.go:47-48). */
MG_API void mongoose_fp32_to_fp16(const float* in, void* out, int n, cudaStream_t stream);
MG_API void mongoose_fp16_to_fp32(const void* in, float* out, int n, cudaStream_t stream);

/* Every layer in [layerStart, layerEnd) for one token, enqueued by one call on `stream`, on
 * caller-owned buffers: per-layer pointer arrays (device addresses held in HOST arrays, as built by
 * BuildFusedDispatch, cuda_fused_infer.go:744-781), raw GGUF Q4_0 weight blocks, fp32 KV caches
 * [maxSeq, kvDim], fp32 norms and scratch vectors.  Signature from cuda_graph.go:211-222; the reference
 * ships no source for it.  Capture-safe: no allocation, no synchronisation. */
MG_API void mongoose_partial_step_q4_fused_graph(
    const float** norm1, const void** wq, const void** wk, const void** wv, const void** wo,
    const float** norm2, const void** wgate, const void** wup, const void** wdown,
    float** kCache, float** vCache,
    float* hidden, float* normed, float* Q, float* K, float* V,
    float* attnOut, float* proj, float* normed2,
    float* gatePre, float* upOut, float* ffnMid,
    void* q8Scratch,
    const float* cosTab, const float* sinTab,
    int dim, int kvDim, int headDim, int ffnDim, int nHeads, int nKVHeads, int halfHead,
    int pos, int layerStart, int layerEnd,
    cudaStream_t stream);

/* Block-32 Q8_0 matvec on raw 34-byte blocks {fp16 d, int8 q[32]}, value d*q.
 * No counterpart in the reference (its INT8 kernel is per-row); provided so the single-op
 * configuration can be driven through caller-owned raw blocks like mongoose_q4_0_matvec. */
MG_API void mongoose_q8_0_matvec(const float* act, const void* w_blocks, float* out, int N, int K,
                          cudaStream_t stream);

/* ------------------------------------------------------------------ */
/* 2. Decode engine                                                    */
/* ------------------------------------------------------------------ */

enum {
    MG_OK = 0,
    MG_ERR_ARG = -1,         /* bad argument (shape, index, NULL) */
    MG_ERR_STATE = -2,       /* call out of order (e.g. step before every weight is set) */
    MG_ERR_CUDA = -3,        /* a CUDA call failed; mg_last_error has the text */
    MG_ERR_NOMEM = -4,
    MG_ERR_UNSUPPORTED = -5,
    MG_ERR_TIMEOUT = -6      /* a bounded device-side wait expired; the context stays usable */
};

/* Weight storage formats. */
enum { MG_FMT_Q8_0 = 0, MG_FMT_Q4_0 = 1, MG_FMT_F16 = 2 };

/* Model description: the positional arguments of NewCUDAFusedInference
 * (cuda_fused_infer.go:144) plus what the reference hard-codes. */
typedef struct mg_config {
    int dim, kv_dim, head_dim, n_heads, n_kv_heads, ffn_dim, vocab, n_layers, max_seq;
    double rope_theta;
    float rms_eps;      /* 0 selects 1e-6, the value at kernels/mongoose.cu:170 */
    int layer_fmt;      /* MG_FMT_* of the seven per-layer matrices */
    int head_fmt;       /* MG_FMT_* of lm_head (also the tied input embedding) */
    int device;         /* CUDA device ordinal */
    int max_batch;      /* independent sequences decoded per step; 0 or 1 = one sequence */
    int flags;          /* reserved, 0 */
} mg_config;

typedef struct mg_engine mg_engine;

/* NewCUDAFusedInference (cuda_fused_infer.go:144-229): allocates activations, KV caches (fp16) and
 * RoPE tables (computed in float64 on the host, cuda_fused_infer.go:181-190). */
MG_API int mg_create(const mg_config* cfg, mg_engine** out);
MG_API void mg_destroy(mg_engine* e);
/* NumWeights (cuda_fused_infer.go:231-233): n_layers*12 + 2. */
MG_API int mg_num_weights(const mg_engine* e);
/* SetWeight (cuda_fused_infer.go:241-272): fp32 tensor for slot idx = layer*12 + w
 * (0 norm1, 1 wq, 2 wk, 3 wv, 4-6 q/k/v bias, 7 wo, 8 norm2, 9 gate, 10 up, 11 down;
 * n_layers*12 final norm; n_layers*12+1 lm_head).  Matrices are quantized on the host to the slot's
 * format, as the reference quantizes in SetWeight; biases are optional. */
MG_API int mg_set_weight(mg_engine* e, int idx, const float* data, size_t count);
/* SetWeightQ4_0 / UploadQ4_0 (cuda_fused_infer_q4.go:46-90, cuda_q4_0.go:15-26): raw blocks of
 * `fmt` (34-byte Q8_0, 18-byte Q4_0, or fp16) for a matrix slot. */
MG_API int mg_set_weight_raw(mg_engine* e, int idx, const void* blocks, size_t bytes, int fmt);
/* BuildFusedDispatch (cuda_fused_infer.go:744-781): checks that every slot is set and prepares the
 * launch sequence.  Called implicitly by the first step. */
MG_API int mg_build(mg_engine* e);
/* ResetKV (cuda_fused_infer.go:530-537); clears K and V. */
MG_API int mg_reset_kv(mg_engine* e);
/* PartialStep (cuda_fused_infer.go:392-459): HOST hidden_in[dim] -> layers [layer_start, layer_end)
 * at position pos -> HOST logits_out[vocab] when the range reaches the last layer and logits_out is
 * not NULL, else HOST hidden_out[dim] when not NULL.  Blocks until the outputs are on the host.
 * A page-locked logits_out (cudaHostAlloc / cudaHostRegister) is filled by the kernel's own stores;
 * pageable memory gets the reference's copy (ToHost, cuda_tensor.go:622). */
MG_API int mg_partial_step(mg_engine* e, const float* hidden_in, int pos, int layer_start, int layer_end,
                    float* hidden_out, float* logits_out);
/* ExportHidden (cuda_fused_infer.go:235-239). */
MG_API int mg_export_hidden(mg_engine* e, float* hidden_out);
/* One greedy step with the tied embedding: token -> every layer -> argmax.  next_token and
 * logits_out (vocab floats, may be NULL) are HOST pointers.  The embedding row is the dequantized
 * row `token` of lm_head. */
MG_API int mg_step_token(mg_engine* e, int token, int pos, int* next_token, float* logits_out);
/* Greedy generation kept on the device: feeds n_prompt tokens one position at a time (the
 * reference has no batched prefill on this path), then n_new greedy steps with the argmax fed back
 * without leaving the GPU.  out_tokens (HOST, n_new ints) receives the generated ids.  start_pos is
 * the position of prompt[0]. */
MG_API int mg_generate(mg_engine* e, const int* prompt, int n_prompt, int n_new, int start_pos,
                int* out_tokens);
/* Enqueue `n_steps` device-resident greedy steps starting from the engine's current device-side
 * token/position without any host synchronisation (benchmark use); mg_sync waits for them. */
MG_API int mg_enqueue_greedy(mg_engine* e, int n_steps);
/* Set the device-side token and position that mg_enqueue_greedy continues from. */
MG_API int mg_set_cursor(mg_engine* e, int token, int pos);
/* Read back the device-side cursor and the last `n` generated tokens (n <= steps since set_cursor). */
MG_API int mg_get_cursor(mg_engine* e, int* token, int* pos);
MG_API int mg_sync(mg_engine* e);
/* Debug/parity: dequantize rows [row0, row0+nrows) of matrix slot idx from the engine's device
 * layout into HOST out[nrows, cols] (value = float(d) * q exactly). */
MG_API int mg_dequant_rows(mg_engine* e, int idx, int row0, int nrows, float* out);
/* Debug/parity: copy fp16 K and V rows [pos0, pos0+npos) of a layer to HOST (uint16 bit patterns). */
MG_API int mg_read_kv(mg_engine* e, int layer, int pos0, int npos, uint16_t* k_out, uint16_t* v_out);
/* Per-phase timeline of ONE greedy step from the current cursor (the counterpart of the reference's
 * per-op [PROFILE] timing at pos 1, cuda_fused_infer_q4.go:147-242).  stamps receives
 * [n_ctas][n_events] SM clock values of each CTA's first thread, n_events = (n_layers + 1) * 32: per
 * layer (lm_head counts as layer n_layers, phase 0), event 2p = input of phase p staged, 2p+1 = phase p
 * done (p: 0 QKV, 1 wo, 2 gate/up, 3 down), 8 = layer start, 9 = attention done (CTAs that run a head),
 * 11+3p = the CTA's tiles of phase p multiplied, 12+3p = all warps past them; other slots unused.
 * Needs the persistent kernel; capacity is in stamps. */
MG_API int mg_trace_step(mg_engine* e, long long* stamps, int capacity, int* n_ctas, int* n_events);
/* Device memory.  An engine reserves ONE device allocation at mg_create, sized from the model's shape,
 * and carves every buffer out of it best-fit in 256-byte units (the reference's GPUArena,
 * gpu_alloc.go:45-241; without it the reference pays one cudaMalloc per tensor, cuda_tensor.go:19-28).
 * The calls below hand pieces of the same arena to the caller: the counterparts of tw_gpu_alloc /
 * tw_gpu_upload / tw_gpu_download / tw_gpu_zero (cuda_tensor.go:19-44) and ArenaStats
 * (gpu_alloc.go:58-66).  A request the arena cannot serve is passed to cudaMalloc (counted in
 * `outside`). */
MG_API int mg_device_alloc(mg_engine* e, size_t bytes, void** out);
MG_API int mg_device_free(mg_engine* e, void* p);
MG_API int mg_device_upload(mg_engine* e, void* dst, const void* host, size_t bytes);
MG_API int mg_device_download(mg_engine* e, void* host, const void* src, size_t bytes);
MG_API int mg_device_zero(mg_engine* e, void* dst, size_t bytes);
MG_API int mg_arena_stats(const mg_engine* e, size_t* total, size_t* in_use, size_t* peak, size_t* largest_free,
                          int* outside);
/* Which decode path a built engine runs (no counterpart in the reference, whose path is fixed): bit 0 the
 * persistent kernel, bit 1 its feed-forward block without an exchange of the middle vector (one GPU),
 * bit 2 tensor-parallel exchange inside the kernels.  0 = the graph of per-phase kernels. */
MG_API int mg_decode_path(const mg_engine* e);
/* Limit of every wait inside the persistent kernel (ring barriers, exchange polls), in milliseconds
 * of SM clock at 2 GHz; the default is about a second.  A wait that runs out makes the step return
 * MG_ERR_TIMEOUT; the context stays usable.  The reference's device-side waits (WaitMailbox,
 * cuda_fused_infer.go:575-590) have no limit at all. */
MG_API int mg_set_wait_limit_ms(mg_engine* e, int ms);
/* ---- replay API (CaptureGraph / Launch / UpdateAndLaunch / ValidateGraphCapture, cuda_graph.go:313-739) ----
 * The reference captures a layer range into a CUDA graph and replays it with the position patched
 * in a device-side parameter block.  Here every step already replays a cached graph (or runs the
 * persistent kernel) and reads its position from device memory, so these calls only expose that:
 * nothing is captured per position and UpdateAndLaunch has nothing to update. */
/* UploadHidden (cuda_graph.go:651): hidden state of the next launch. */
MG_API int mg_upload_hidden(mg_engine* e, const float* hidden);
/* CUDAGraph.Launch(pos) (cuda_graph.go:663-671): layers [layer_start, layer_end) at `pos` on the
 * device-resident hidden state; asynchronous, no host copies.  Read the result with mg_export_hidden. */
MG_API int mg_graph_launch(mg_engine* e, int pos, int layer_start, int layer_end);
/* ValidateGraphCapture (cuda_graph.go:554-601): the range at position 0 through plain one-by-one
 * kernel launches and through the replay path; max_diff receives the largest absolute difference of
 * the two hidden states (the reference accepts < 1e-3).  Resets the KV cache. */
MG_API int mg_validate_replay(mg_engine* e, const float* hidden_in, int layer_start, int layer_end, float* max_diff);

/* ---- layer-range pipeline (SetLayerRange, PartialStepContinue, QueueHiddenToL3, WaitL3, WaitMailbox;
 * cuda_fused_infer.go:461-737) ----------------------------------------------------------------------
 * A stage is an engine that holds a contiguous range of layers (the last stage also the final norm and
 * lm_head).  The reference hands the hidden state from stage to stage through a pinned host buffer
 * ("L3 bridge") and a mailbox counter polled without a time limit; here the hand-over between GPUs of
 * one process is a peer copy over NVLink ordered by events, and every host-side wait has a deadline. */
/* SetLayerRange (cuda_fused_infer.go:542-556): only these layers need weights; steps outside fail. */
MG_API int mg_set_layer_range(mg_engine* e, int layer_start, int layer_end);
/* PartialStepContinue (cuda_fused_infer.go:463-528): PartialStep on the hidden state already on the
 * device (uploaded, left by the previous range, or queued by the previous stage). */
MG_API int mg_partial_step_continue(mg_engine* e, int pos, int layer_start, int layer_end, float* hidden_out,
                                    float* logits_out);
/* Hands src's device-resident hidden state to dst (another GPU: cudaMemcpyPeerAsync) on src's stream
 * and makes dst's stream wait for it; asynchronous. */
/* StepLayerResident (cuda_fused_infer_q4.go:451-605): ONE layer at position pos, with HOST snapshots of
 * the hidden state before (pre_out) and after (post_out) it; layer 0 uploads hidden_in, later layers
 * continue on the device-resident hidden state; logits_out (any layer, as in the reference) adds the
 * final norm and lm_head on the layer's output.  Any of the three outputs may be NULL. */
MG_API int mg_step_layer_resident(mg_engine* e, int layer, int pos, const float* hidden_in, float* pre_out,
                                  float* post_out, float* logits_out);
/* vNodes (SetVNodeCount / RecordStageDone / WaitStageDone / SyncStream1 / QueueHiddenToL3OnStream1 /
 * PartialStepQ4ContinueOnStream1, cuda_fused_infer.go:630-684, cuda_fused_infer_q4.go:391-444).  The
 * reference overlaps two pipeline stages of one GPU on two compute streams; here a stage is one
 * persistent launch over every SM, so "stream 1" is an ordering domain only: the calls keep their
 * names, their order and their results, the stages run one after the other. */
MG_API int mg_set_vnode_count(mg_engine* e, int n);
MG_API int mg_vnode_count(const mg_engine* e);
MG_API int mg_record_stage_done(mg_engine* e);
MG_API int mg_wait_stage_done(mg_engine* e);
MG_API int mg_sync_stream1(mg_engine* e);
MG_API int mg_partial_step_continue_on_stream1(mg_engine* e, int pos, int layer_start, int layer_end, float* logits_out);
MG_API int mg_queue_hidden_to_l3_on_stream1(mg_engine* e);
MG_API int mg_queue_hidden_to(mg_engine* src, mg_engine* dst);
/* WaitMailbox (cuda_fused_infer.go:575-591) with a deadline: MG_OK once the hidden state last queued
 * to e has arrived, MG_ERR_TIMEOUT after timeout_ms (also when nothing was queued). */
MG_API int mg_wait_mailbox(mg_engine* e, int timeout_ms);
/* QueueHiddenToL3 / WaitL3 / GetL3Hidden (cuda_fused_infer.go:686-726): asynchronous copy of the hidden
 * state to a pinned host buffer on a second stream; the compute stream is not blocked. */
MG_API int mg_queue_hidden_to_l3(mg_engine* e);
MG_API int mg_wait_l3(mg_engine* e, int timeout_ms);
MG_API const float* mg_l3_hidden(mg_engine* e);

/* ---- tensor-parallel decode over 2/4/8 GPUs of one node, one process per GPU ----------------------
 * The reference has no tensor parallelism (multigpu.go:32-82, 496-623 manages per-device handles and
 * peer copies only); these calls split one model over ranks.  QKV, gate and up are split by rows at
 * whole-head granularity, wo and down by columns (partial sums), lm_head by vocabulary rows; the KV
 * cache follows its heads.  Per token: two all-reduces of dim fp32 per layer, one all-reduce of the
 * packed (logit, index) argmax key, and an all-gather of logits when logits are asked for.
 * Every rank calls mg_set_weight / mg_set_weight_raw with the FULL tensor and keeps its part. */
typedef struct mg_tp_shard {
    int q_head0, q_head1;     /* query heads [q_head0, q_head1) */
    int kv_head0, kv_head1;   /* KV heads that serve them (a KV head may be replicated on several ranks) */
    int ffn0, ffn1;           /* FFN features, multiples of 32 */
    int vocab0, vocab1;       /* lm_head rows */
} mg_tp_shard;
/* The partition rank `rank` of `size` would hold; pure host arithmetic, needs no GPU.
 * MG_ERR_UNSUPPORTED when the KV heads neither divide among the ranks nor are divided by them. */
MG_API int mg_tp_partition(const mg_config* cfg, int rank, int size, mg_tp_shard* out);
/* A fresh 128-byte communicator id (rank 0 makes it and hands it to the other ranks by any means). */
MG_API int mg_tp_unique_id(void* id_out, size_t bytes);
/* Joins the communicator; collective over all ranks.  Call once, after mg_create and before any
 * weight is set.  NCCL is resolved from libnccl.so.2 at this point, not at load time. */
MG_API int mg_tp_init(mg_engine* e, int rank, int size, const void* id, size_t bytes);
/* The stream the engine enqueues on (for event timing by the caller). */
/* Test aid (no counterpart in the reference): rank 0 of a `size`-rank tensor-parallel group whose peers
 * do not exist, on one GPU.  Nothing ever writes the other ranks' rows of the receive buffer, so the
 * first in-kernel wait for them runs out after the wait limit and the step returns MG_ERR_TIMEOUT with
 * the exchange named in mg_last_error: the way to exercise the bounded device-side waits without a
 * second GPU and without faulting or hanging one. */
MG_API int mg_tp_init_absent_peers(mg_engine* e, int size);
MG_API cudaStream_t mg_stream(mg_engine* e);
/* Kernels launched by this engine since creation (graph replays count their kernel nodes). */
MG_API long long mg_launch_count(const mg_engine* e);
/* Device bytes held by the engine. */
MG_API size_t mg_device_bytes(const mg_engine* e);
/* Text of the last error on this engine (never NULL). */
MG_API const char* mg_last_error(const mg_engine* e);
/* Library build description, e.g. "mongoose-b200 sm_100a". */
MG_API const char* mg_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MONGOOSE_KERNELS_H */
