/* b200gpt — C ABI of the B200-native (sm_100a) quantized-decode hot path of lit-gpt.
 *
 * Every entry point takes raw DEVICE pointers, sizes and a CUDA stream (`cudaStream_t` passed as void*),
 * launches asynchronously on that stream, never allocates, never synchronises, and returns 0 on success.
 * On failure it returns a B200_ERR_* code and `b200_last_error()` (thread-local) holds the message.
 * Caller-owned workspaces are sized by the *_workspace_bytes helpers.
 *
 * Each function cites the reference interface it replaces (file:line into yuanyaaa/lit-gpt).  The reference's
 * own quantized arithmetic lives in bitsandbytes==0.41.0 (requirements-all.txt:3) behind
 * lightning.fabric.plugins.BitsandbytesPrecision (generate/base.py:129-134); see INTEGRATION.md for the
 * binding a maintainer would add.
 */
#ifndef B200GPT_H
#define B200GPT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200GPT_ABI_VERSION 1

typedef void* b200_stream_t; /* cudaStream_t */

enum b200_status { B200_OK = 0, B200_ERR_INVALID = 1, B200_ERR_CUDA = 2, B200_ERR_UNSUPPORTED = 3 };
enum b200_dtype { B200_BF16 = 0, B200_F16 = 1, B200_F32 = 2 };
/* 4-bit weight formats.  NF4/FP4: bitsandbytes block-64 codebooks; INT4: this project's group-128 format
 * (the reference has no gptq/int4 code). */
enum b200_qtype { B200_Q_NF4 = 0, B200_Q_FP4 = 1, B200_Q_INT4 = 2 };
/* GEMV epilogues */
enum b200_epilogue { B200_EPI_STORE = 0, B200_EPI_RESIDUAL = 1, B200_EPI_SWIGLU = 2 };

/* ---- library ------------------------------------------------------------------------------------------ */
int b200_abi_version(void);
const char* b200_last_error(void);
/* fills SM count and compute capability of the current device */
int b200_device_info(int* sm_count, int* cc_major, int* cc_minor);
/* enable/disable programmatic dependent launch (griddepcontrol) on every kernel of the library; returns old value */
int b200_set_pdl(int enabled);
/* number of kernels launched by this library since load (the `gpu_launches` evidence of bench.py) */
int64_t b200_launch_count(void);
/* tuning override for the fast GEMV: ksteps in {0(auto),1,2,4}, ctas_per_sm in {0(auto),1,2,3,4}; returns 0 */
int b200_qgemv_tune(int ksteps, int ctas_per_sm, int force_generic);

/* ---- quantisation (replaces bitsandbytes.functional.quantize_4bit / dequantize_4bit reached through
 *      Params4bit.cuda(); reference call sites generate/base.py:168, generate/tp.py:190, lit_gpt/lora.py:156-160) */
/* w: `numel` elements of w_dtype, flattened row-major.  packed: (numel+1)/2 bytes, even element in the HIGH
 * nibble.  absmax: ceil(numel/blocksize) floats.  qtype NF4|FP4.  blocksize must be even (reference uses 64). */
int b200_quantize_4bit(const void* w, int w_dtype, int64_t numel, int blocksize, int qtype, uint8_t* packed,
                       float* absmax, b200_stream_t stream);
int b200_dequantize_4bit(const uint8_t* packed, const float* absmax, int64_t numel, int blocksize, int qtype,
                         void* out, int out_dtype, b200_stream_t stream);
/* Double quantisation of an absmax vector (--quantize bnb.nf4-dq / bnb.fp4-dq; bitsandbytes quantize_4bit with
 * compress_statistics=True, reference call sites generate/base.py:105,129-134): blocks of 256, `offset` (the mean,
 * computed by the caller) is subtracted, block absmax -> absmax2, 8-bit index into the 256-entry dynamic code
 * (code256, sorted ascending) -> q_out, and absmax_deq_out = code[q] * absmax2 + offset, the value every later
 * dequantise / GEMV of the layer uses.  n values in, ceil(n / 256) absmax2 out. */
int b200_double_quant_absmax(const float* absmax, int64_t n, const float* code256, float offset, uint8_t* q_out, float* absmax2_out,
                             float* absmax_deq_out, b200_stream_t stream);

/* int4 group-128 (asymmetric RTN, GPTQ storage order): qweight uint32 (N, ceil(K/8)), scales fp16 (N, G),
 * qzeros uint32 (N, ceil(G/8)), G = ceil(K/group).  `sz` (optional, may be NULL) receives the kernel-side
 * interleaved half2 {scale, zero} per (row, group) that b200_qgemv consumes. */
int b200_quantize_int4(const void* w, int w_dtype, int64_t N, int64_t K, int group, uint32_t* qweight,
                       uint16_t* scales, uint32_t* qzeros, uint32_t* sz, b200_stream_t stream);
int b200_dequantize_int4(const uint32_t* qweight, const uint16_t* scales, const uint32_t* qzeros, int64_t N,
                         int64_t K, int group, void* out, int out_dtype, b200_stream_t stream);

/* ---- fused dequant-GEMV, batch 1..16 (replaces bnb.nn.Linear4bit.forward -> kgemm_4bit_inference_naive /
 *      dequantize+F.linear at lit_gpt/model.py:619,656,713,714,716,519) ------------------------------------
 * y[b, n] = epilogue( sum_k xin[b, k] * W[n, k] ),  xin = prologue(x):
 *   prologue: xin = x (+ delta if delta != NULL, rounded to bf16); if x_out != NULL the summed rows are written
 *             there by one CTA (x_out must not alias x); if norm_weight != NULL xin = RMSNorm(xin) with
 *             lit_gpt/rmsnorm.py:19-25 rounding (fp32 math, one cast).
 *   W:        qtype NF4/FP4: `packed` + `absmax` (blocksize 64) as produced by b200_quantize_4bit on the
 *             row-major (N, K) weight; INT4: qweight + sz.  For B200_EPI_SWIGLU a second matrix (packed2/scale2)
 *             of the same shape is given and y[b,n] = silu(W·xin) * (W2·xin) with the reference's bf16 rounding
 *             points (lit_gpt/model.py:712-716).
 *   epilogue: STORE: y = acc (+ bias); RESIDUAL: y = bf16(acc + bias) + residual (lit_gpt/model.py:591-592).
 * x, delta, x_out, residual, y, bias, norm_weight are bf16.  batch <= 16.  workspace: b200_qgemv_workspace_bytes().
 */
typedef struct b200_qgemv_args {
  const void* packed;     /* uint8 (NF4/FP4) or uint32 (INT4) */
  const void* scale;      /* float absmax (NF4/FP4) or half2 sz (INT4) */
  const void* packed2;    /* second matrix for SWIGLU, else NULL */
  const void* scale2;
  int qtype;
  int blocksize;          /* 64 for NF4/FP4, 128 for INT4 */
  int64_t N, K;
  const void* x;          /* (batch, K) bf16 */
  const void* delta;      /* optional (batch, K) bf16 */
  void* x_out;            /* optional (batch, K) bf16 */
  const void* norm_weight;/* optional (K) bf16 */
  float norm_eps;
  int batch;
  int epilogue;
  const void* bias;       /* optional (N) bf16 */
  const void* residual;   /* (batch, N) bf16 for EPI_RESIDUAL; may alias y */
  void* y;                /* (batch, N) bf16 */
  void* workspace;
  size_t workspace_bytes;
} b200_qgemv_args;
size_t b200_qgemv_workspace_bytes(void);
int b200_qgemv(const b200_qgemv_args* args, b200_stream_t stream);

/* ---- tiled weight layout + streaming GEMV (the decode hot path; csrc/tile.cu, csrc/qgemv_stream.cu) -----------
 * b200_tile_4bit permutes the reference-layout arrays (packed + absmax of b200_quantize_4bit, or qweight + sz of
 * b200_quantize_int4) into per-(16-row tile, 64-wide k-block) records laid out in warp-consumption order;
 * b200_untile_4bit is the exact inverse (so the bitsandbytes-layout bytes are always recoverable bit for bit).
 * K must be a multiple of 64 (NF4/FP4, blocksize 64) or 128 (INT4, group 128).  b200_tiled_bytes returns 0 for
 * shapes the layout does not cover. */
size_t b200_tiled_bytes(int64_t N, int64_t K, int qtype);
int b200_tile_4bit(const void* packed, const void* scale, int64_t N, int64_t K, int qtype, int blocksize, void* tiled,
                   b200_stream_t stream);
int b200_untile_4bit(const void* tiled, int64_t N, int64_t K, int qtype, int blocksize, void* packed, void* scale,
                     b200_stream_t stream);
/* Same contract as b200_qgemv (prologue / epilogues / rounding points), reading tiled matrices; no workspace.
 * `prefetch`/`prefetch_bytes` (optional): a range the kernel asks the L2 to fetch (cp.async.bulk.prefetch.L2) -
 * the weights of the NEXT kernel in the decode graph - so HBM stays busy across the kernel boundary. */
/* Tensor-parallel hand-off fused into the GEMV (replaces the all_reduce hook of generate/tp.py:73-74 on the decode path;
 * DESIGN.md §6).  PRODUCER = the row-parallel Linear (attn.proj, mlp.proj): its epilogue stores this rank's partial
 * into slot `rank` of EVERY rank's buffer over NVLink peer memory as self-validating 32-bit packets
 * `tag << 16 | bf16 bits` (one store per output element, no fence, no separate flag: the "LL" scheme).
 * CONSUMER = the next Linear (whose `delta` the all-reduced tensor would have been): its prologue polls the `world`
 * local slots until every packet carries the expected tag, adds them in rank order in fp32, rounds once to bf16 and
 * carries on as with `delta`; its last CTA bumps the buffer's sequence counter.  tag = seq % 65535 + 1, where seq is
 * the buffer's LOCAL counter (all ranks run the same launch sequence, so the counters stay in lock step).
 * Consecutive hand-offs must alternate between two buffers.  Counters are uint32 and zero before first use, slots are
 * zero before first use.  Pointers come from b200_p2p_alloc / b200_p2p_open. */
typedef struct b200_tp_handoff {
  int world, rank;
  void* peer_y[8];        /* producer: slot `rank` (batch, N) uint32 packets in the buffer of rank r, own rank included */
  void* reduced;          /* consumer, optional: LOCAL buffer of >= batch * K uint32 packets.  When set the exchange is summed in two
                             stages: every CTA adds the `world` slots for ITS slice of the vector only and republishes the sums here as
                             packets with the same tag, then all CTAs read this one buffer: world x fewer L2 reads per CTA (at world 8
                             each CTA otherwise reads 8 x K x 4 bytes), one more local round trip.  Same arithmetic, bit-identical. */
  void* reserved[7];      /* must be NULL */
  void* send_seq;         /* producer: LOCAL sequence counter of the buffer written; NULL = this launch is not a producer */
  const void* slots;      /* consumer: local slots, rank r at slots + r * slot_stride bytes; NULL = not a consumer */
  int64_t slot_stride;    /* >= batch * K * 4 bytes */
  void* recv_seq;         /* consumer: LOCAL sequence counter of the buffer read (bumped by the launch's last CTA) */
  void* recv_done;        /* consumer: local CTA counter */
} b200_tp_handoff;
/* All-gather over the same slots (`lm_head` sharded by rows under tensor parallelism; the reference replicates it,
 * generate/tp.py:77-80).  The sharded Linear's GEMV is launched as a PRODUCER (tp->send_seq / peer_y set, y may be NULL): rank r's
 * (batch, N / world) outputs land in slot r of every rank's gather buffer.  This call is the CONSUMER: it polls the `world` slots of
 * the local buffer (consumer fields of `h`), unpacks them into out (batch, world * n_per_rank) bf16 in rank order -- i.e. the
 * unsharded Linear's output -- and bumps the buffer's sequence counter.  The gather buffer is a third hand-off buffer with its own
 * counters (it must not be one of the two alternating branch buffers).  error_word: optional, set to 2 on a bounded-wait time-out. */
int b200_tp_gather(const b200_tp_handoff* h, int batch, int64_t n_per_rank, void* out, void* error_word, b200_stream_t stream);
/* Symmetric peer buffers (setup time, not per token): cudaMalloc + zero + IPC export / import / release. */
int b200_p2p_alloc(size_t bytes, void** ptr, void* handle64);
int b200_p2p_open(const void* handle64, void** ptr);
int b200_p2p_close(void* ptr);
int b200_p2p_free(void* ptr);

/* Optional hint for the launch that precedes a decode-attention step (the fused QKV projection): once its own weight stream
 * has been issued, the kernel asks the L2 for the filled part of this layer's K / V cache (cp.async.bulk.prefetch.L2), so that
 * the attention kernel's dependent loads hit L2 instead of HBM.  `chunks` = batch * n_query_groups contiguous (Tmax, hs) planes
 * per tensor, `chunk_stride` bytes apart; rows [0, *pos) of `row_bytes` each are fetched.  A hint only: no effect on results. */
struct b200_attn_decode_args;
typedef struct b200_kv_hint {
  const void* k;
  const void* v;
  const void* pos;       /* device scalar, int32 or int64 */
  int pos_is_int64;
  int chunks;
  int64_t chunk_stride;
  int row_bytes;
  int max_rows;
} b200_kv_hint;

typedef struct b200_qgemv_tiled_args {
  const void* tiled;
  const void* tiled2;      /* second matrix for SWIGLU, else NULL */
  int qtype;
  int blocksize;           /* 64 for NF4/FP4, 128 for INT4 */
  int64_t N, K;
  const void* x;           /* (batch, K) bf16 */
  const void* delta;       /* optional (batch, K) bf16 */
  void* x_out;             /* optional (batch, K) bf16 */
  const void* norm_weight; /* optional (K) bf16 */
  float norm_eps;
  int batch;
  int epilogue;
  const void* bias;        /* optional (N) bf16 */
  const void* bias2;       /* optional (N) bf16, SWIGLU second matrix */
  const void* residual;    /* (batch, N) bf16 for EPI_RESIDUAL; may alias y */
  void* y;                 /* (batch, N) bf16 */
  const void* prefetch;
  int64_t prefetch_bytes;
  void* workspace;         /* zero-initialised once by the caller, >= b200_qgemv_tiled_workspace_bytes(); holds the
                              partial sums / arrival counters of row pairs cut by a stream-K boundary (self-cleaning) */
  size_t workspace_bytes;
  const struct b200_tp_handoff* tp; /* optional tensor-parallel hand-off (below); NULL on one GPU */
  const b200_kv_hint* kv_hint; /* optional (above); NULL = none */
  const struct b200_attn_decode_args* attn; /* optional: the decode-attention step that consumes this launch's output, FUSED into
                              the same kernel (replaces lit_gpt/model.py:619 + 624-653 with one launch): y is the interleaved QKV row,
                              attn->qkv must equal y, attn->out receives (1, n_head * head_size).  Batch 1, n_head == n_query_groups,
                              head size 128, STORE epilogue; each head's attention runs on the CTA of the same index as soon as the
                              head's q / k / v rows are stored (per-head counters in the workspace), four key ranges on four
                              128-thread sub-blocks merged in shared memory.  Anything else: B200_ERR_UNSUPPORTED, nothing launched
                              (call b200_attn_decode separately).  attn->workspace is not used. */
  int fold;                /* 0 / 1: plain.  F = 2, 4: `tiled` holds the matrix VIEWED as (N / F, F * K), i.e. b200_tile_4bit(N / F, F * K)
                              of the same flat nf4 / fp4 buffers: for row-parallel shards whose K is not a multiple of the
                              64-element block while F * K is (generate/tp.py:28-45 cuts mlp.proj to 11008 / 8 = 1376 columns, and
                              bitsandbytes quantizes the shard's FLAT storage, so blocks straddle rows).  N, K, x and y keep the
                              true shapes; STORE / RESIDUAL epilogues, no norm / delta / tp consumer, batch * F <= 16. */
} b200_qgemv_tiled_args;
/* 1 when b200_qgemv_tiled would run these arguments on a streaming kernel, 0 when the shape is outside every plan (nothing
 * is launched, pointers are not dereferenced): lets the caller choose the generic b200_qgemv / b200_qgemm up front. */
int b200_qgemv_tiled_supported(const b200_qgemv_tiled_args* args);
/* Bounded waits instead of hangs or traps: a kernel that waited ~2 s for a partner (a tensor-parallel peer's packets, a
 * stream-K partner CTA) sets word 0 of the workspace and carries on.  This call synchronizes `stream`, returns the word in
 * *code (0 = none, 1 = stream-K partner, 2 = tensor-parallel peer) and clears it.  generate() checks it at its sync points. */
int b200_qgemv_tiled_error(void* workspace, b200_stream_t stream, unsigned int* code);
size_t b200_qgemv_tiled_workspace_bytes(void);
int b200_qgemv_tiled(const b200_qgemv_tiled_args* args, b200_stream_t stream);
/* tuning: depth in {0(auto),2,4,6} items loaded ahead per warp; ctas_per_sm in {0(auto),1,2}; l2_prefetch 0/1 */
int b200_qgemv_tiled_tune(int depth, int ctas_per_sm, int l2_prefetch);
/* diagnostics (no counterpart in the reference): the next `slots` b200_qgemv_tiled launches record eight per-CTA phase time
 * stamps (%globaltimer, ns) into buf[slots][160][8] (uint64, device memory, caller-owned, zeroed by the caller);
 * buf = NULL switches it off.  tools/trace_step.py turns them into the per-launch timeline quoted in DESIGN.md. */
int b200_qgemv_tiled_trace(void* buf, int slots);

/* ---- RMSNorm (replaces lit_gpt/rmsnorm.py:19-25 and the residual add at lit_gpt/model.py:591) ------------
 * y = RMSNorm(x (+ delta)) * weight; if sum_out != NULL it receives bf16(x + delta).  rows x dim, bf16. */
int b200_rmsnorm(const void* x, const void* delta, const void* weight, float eps, void* y, void* sum_out,
                 int64_t rows, int64_t dim, b200_stream_t stream);

/* ---- fused RoPE + KV-cache append + split-K flash-decode attention, T = 1 (replaces lit_gpt/model.py:624-653:
 *      view/permute/split, apply_rope 767-773, KVCache.forward 788-795, scaled_dot_product_attention 658-665)
 * qkv: (batch, (n_head + 2*n_groups) * head_size) bf16 in the reference's per-group interleaved order
 *      [q * q_per_kv, k, v] x n_groups (lit_gpt/model.py:621-628).
 * cos/sin: the model's own tables (max_seq, rope_n_elem), fp32 or bf16 (never recomputed in-kernel).
 * pos: device int64/int32 scalar = position being written (input_pos); keys 0..pos are attended.
 * k_cache/v_cache: (batch, n_groups, max_seq, head_size) bf16, GQA-native (n_groups heads).
 * out: (batch, n_head * head_size) bf16.  head_size in {64, 128}. */
typedef struct b200_attn_decode_args {
  const void* qkv;
  const void* cos;
  const void* sin;
  int table_dtype;   /* B200_F32 or B200_BF16 */
  int table_preselected; /* 1: cos/sin point at the row already gathered for this token (model.py:505-506); 0: full tables indexed by pos */
  int rope_n_elem;
  const void* pos;   /* device scalar */
  int pos_is_int64;
  void* k_cache;
  void* v_cache;
  void* out;
  int batch, n_head, n_groups, head_size, max_seq;
  int num_splits;    /* 0 = auto */
  void* workspace;
  size_t workspace_bytes;
} b200_attn_decode_args;
size_t b200_attn_decode_workspace_bytes(int batch, int n_head, int head_size, int max_splits);
int b200_attn_decode(const b200_attn_decode_args* args, b200_stream_t stream);
/* development / test knob: 1 = always use the scalar kernel with the workspace merge, even for grouped-query shapes that
 * the mma.sync kernel covers (head_size 128, 2 <= q_per_kv <= 16) and for split counts <= 8 that would otherwise run as a
 * thread-block cluster merging through distributed shared memory.  Returns the previous setting. */
int b200_attn_decode_tune(int force_scalar);

/* Allocation-free variant of b200_attn_decode.  It has NO counterpart in the reference: it was added at the request of the
 * run's operators for callers that cannot call cudaMalloc (code under CUDA graph capture, tight serving loops, harnesses
 * that forbid it).  Same arguments and results as b200_attn_decode, except that `workspace` / `workspace_bytes` are
 * ignored: the split-K scratch lives in a static device array of b200_attn_decode_noalloc_max_bytes() = 4 MiB that every
 * GPU loading the library holds until exit.  Shapes whose scratch need
 * b200_attn_decode_workspace_bytes(batch, n_head, head_size, num_splits ? num_splits : 64) exceeds that are rejected with
 * B200_ERR_UNSUPPORTED and a message.  No cudaMalloc / cudaFree / allocating routine is called; one cudaMemsetAsync on
 * `stream` clears the counters that must start at zero.  All calls share the array: calls that overlap on the GPU
 * (different streams, or different threads on different streams) race; calls on one stream are ordered and safe. */
size_t b200_attn_decode_noalloc_max_bytes(void);
int b200_attn_decode_noalloc(const b200_attn_decode_args* args, b200_stream_t stream);

/* ---- prefill helper: RoPE + KV-cache write for T > 1 tokens at positions pos[0..T) (lit_gpt/model.py:624-649).
 * table_preselected = 1: cos/sin are (T, rope_n_elem) rows already gathered by input_pos; 0: full tables.
 * Writes roped q to q_out (batch, n_head, T, head_size) and the roped k / v rows into the GQA-native caches. */
int b200_rope_kv_append(const void* qkv, const void* cos, const void* sin, int table_dtype, int table_preselected,
                        int rope_n_elem, const void* pos, int pos_is_int64, void* k_cache, void* v_cache, void* q_out, int batch,
                        int T, int n_head, int n_groups, int head_size, int max_seq, b200_stream_t stream);

/* ---- prefill attention (T > 1) over the GQA-native caches: replaces F.scaled_dot_product_attention at
 * lit_gpt/model.py:658-665 for the cached multi-token call (model.py:646-650).  q is (batch, n_head, T, head_size),
 * already roped (b200_rope_kv_append); query row t attends to cache positions j <= pos[t] (the mask row
 * model.py:509 selects), so the caches must already hold positions up to max(pos).  fp32 online softmax.
 * y is written as (batch, T, n_head * head_size), the layout attn.proj consumes (model.py:653).
 * head_size 64 or 128. */
int b200_attn_prefill(const void* q, const void* k_cache, const void* v_cache, const void* pos, int pos_is_int64, void* y,
                      int batch, int T, int n_head, int n_groups, int head_size, int max_seq, float scale,
                      b200_stream_t stream);

/* ---- small glue kernels so a whole decode step is one CUDA graph of this library's kernels ---------------- */
/* out[r, :] = wte[idx[r], :]  (lit_gpt/model.py:515) */
/* y = silu(a) * b over n bf16 elements (replaces `F.silu(x_fc_1) * x_fc_2`, lit_gpt/model.py:715, on the prefill path; the decode GEMV
 * has it as its SWIGLU epilogue).  Same rounding points as the reference's two ATen kernels: silu to bf16, product to bf16. */
int b200_swiglu(const void* a, const void* b, void* y, int64_t n, b200_stream_t stream);
int b200_embedding(const void* idx, int idx_is_int64, const void* wte, void* out, int64_t rows, int64_t dim,
                   int64_t vocab, b200_stream_t stream);
/* greedy sampling: token[b] = argmax(logits[b, :vocab]) (generate/base.py:41).  If pos_inout != NULL: pos += 1
 * (generate/base.py:92) and, if history != NULL, history[pos] = token[0] (the torch.cat of generate/base.py:93
 * done on the device), so a whole decode loop needs no host round trip. */
int b200_argmax(const void* logits, int64_t batch, int64_t vocab, int64_t stride, void* token_out,
                int token_is_int64, void* pos_inout, int pos_is_int64, void* history, int64_t history_len,
                b200_stream_t stream);
/* stochastic sampling of batch row 0: sample() / multinomial_num_samples_1() of generate/base.py:22-41 as one launch.
 * logits: vocab values (bf16 or fp32).  top_k <= 0 or >= vocab: no truncation, else only the top_k largest logits are
 * kept (ties at the threshold in index order).  temperature > 0: token = argmax_i softmax(l / T)_i / e_i with
 * e_i ~ Exp(1) (the draw the reference uses under torch.compile, base.py:23-26); temperature <= 0: argmax.
 * rng_state: device int64[2] = {seed, offset}; e_i comes from Philox4x32-10(seed, offset, i) and offset is advanced
 * by one per call (so a captured CUDA graph draws fresh numbers on every replay).  noise (optional, fp32[vocab]):
 * use these Exp(1) values instead (tests).  token / pos / history bookkeeping exactly as b200_argmax. */
int b200_sample(const void* logits, int logits_dtype, int64_t vocab, float temperature, int top_k, void* rng_state,
                const void* noise, void* token_out, int token_is_int64, void* pos_inout, int pos_is_int64, void* history,
                int64_t history_len, b200_stream_t stream);

/* ---- prefill GEMM: y (M, N) = x (M, K) · dequant(W)^T, tcgen05/TMEM mainloop (replaces dequantize_4bit +
 *      F.linear for T > 1 at the same call sites).  Implemented in csrc/qgemm_tcgen05.cu. */
typedef struct b200_qgemm_args {
  const void* packed;
  const void* scale;
  int qtype;
  int blocksize;
  int64_t M, N, K;
  const void* x; /* (M, K) bf16 */
  const void* bias;
  void* y;       /* (M, N) bf16 */
  void* workspace;
  size_t workspace_bytes;
} b200_qgemm_args;
size_t b200_qgemm_workspace_bytes(int64_t M, int64_t N, int64_t K);
int b200_qgemm(const b200_qgemm_args* args, b200_stream_t stream);
/* tuning: mt3 = 1 (default): prompts of more than 512 tokens share each dequantised weight tile among 384 tokens (three 128-row
 * accumulators in tensor memory, three 64 KB stages); 0: 256 tokens as in round 1 */
int b200_qgemm_tune(int mt3);

/* ---- bnb.int8: LLM.int8() inference Linear (replaces bitsandbytes.nn.Linear8bitLt(has_fp16_weights=False,
 *      threshold=6.0) installed by BitsandbytesPrecision("int8") at generate/base.py:129-134; arithmetic restated in
 *      oracle/quant_ref.py:310-345).  Implemented in csrc/int8.cu.
 *      b200_quantize_int8: CB = rint(W * 127 / absmax_row) int8 (N, K), SCB = absmax_row fp32 (N).
 *      b200_linear_int8:   y (M, N) fp16 = LLM.int8()(x (M, K) fp16): outlier columns (any |x| >= threshold) through an
 *      fp16 side product, the rest int8 x int8 -> int32 on the tensor cores.  K must be a multiple of 64
 *      (else B200_ERR_UNSUPPORTED).  The workspace holds the quantised activations; nothing is allocated inside. */
int b200_quantize_int8(const void* w, int w_dtype, int64_t N, int64_t K, int8_t* cb, float* scb, b200_stream_t stream);
int b200_dequantize_int8(const int8_t* cb, const float* scb, int64_t N, int64_t K, void* out, int out_dtype, b200_stream_t stream);
typedef struct b200_linear_int8_args {
  const void* x;      /* (M, K) fp16 */
  const void* cb;     /* (N, K) int8 */
  const void* scb;    /* (N) fp32 */
  const void* bias;   /* (N) fp16 or NULL */
  void* y;            /* (M, N) fp16 */
  int64_t M, N, K;
  float threshold;    /* 6.0 in the reference; <= 0 disables the outlier path */
  void* workspace;
  size_t workspace_bytes;
} b200_linear_int8_args;
size_t b200_linear_int8_workspace_bytes(int64_t M, int64_t K);
int b200_linear_int8(const b200_linear_int8_args* args, b200_stream_t stream);


/* ---- models with an fp32 residual stream, latent attention and sparse experts --------------------------------
 * (no counterpart in the reference, whose models keep the residual in the compute dtype, cache full keys and values and
 * whose only expert layer is the dense-routed LLaMAMoE of lit_gpt/model.py).  `dtype` is the matrix-product dtype of
 * weights and activations, B200_BF16 or B200_F32; statistics, softmax, router and the residual are fp32 in both. */
/* x[row] = embed[tokens[row]] * scale + pos_table[pos[row]] (fp32), act[row] = dtype(x[row]); pos_table may be NULL */
int b200_embed_pos(const int32_t* tokens, const int32_t* pos, const void* embed, const void* pos_table, float scale, float* x,
                   void* act, int64_t rows, int d, int vocab, int max_pos, int dtype, b200_stream_t stream);
/* out[out_rows[i]] = in[in_rows[i]] / sqrt(mean(in^2) + eps) * (weight, or 1 + weight when plus_one); NULL index arrays
 * mean i itself, an out row < 0 is skipped.  One or two segments per launch (e.g. the two halves of a fused projection,
 * the second scattered straight into a cache). */
typedef struct b200_rms_rows_seg {
  const void* in;
  const void* weight;
  void* out;
  const int64_t* in_rows;
  const int64_t* out_rows;
  int64_t ld_in, ld_out;
  int d, plus_one;
} b200_rms_rows_seg;
int b200_rms_rows(const b200_rms_rows_seg* segs, int n_segs, int64_t rows, float eps, int in_dtype, int out_dtype, b200_stream_t stream);
/* x[row] += y[row] / sqrt(mean(y[row]^2) + eps) * (1 + weight); act[row] = dtype(x[row]) */
int b200_residual_norm_add(const void* y, const void* weight, float eps, float* x, void* act, int64_t rows, int d, int dtype,
                           b200_stream_t stream);
/* dst[i] = src[rows[i]]; rows int64 or int32 */
int b200_gather_rows(const void* src, const void* rows, int rows_is_int64, void* dst, int64_t n_rows, int d, int dtype, b200_stream_t stream);
/* x = relu(x)^2 in place over n elements */
int b200_sqrelu(void* x, int64_t n, int dtype, b200_stream_t stream);
int b200_scale_f32(const void* in, float scale, float* out, int64_t n, int dtype, b200_stream_t stream);

/* Ragged causal attention with separate query-key (dk) and value (dv) sizes and no rotation.  seqs[s] = {first query row,
 * query rows, position of the first query row, row of position 0 in k / v}; query row i of sequence s sees key rows
 * kv0 .. kv0 + pos0 + i.  q (rows, n_head * dk), k (.., n_head * dk), v (.., n_head * dv), out (rows, n_head * dv), each
 * with its own leading dimension. */
typedef struct b200_latent_prefill_args {
  const void* q; const void* k; const void* v; void* out;
  int64_t ldq, ldk, ldv, ldo;
  const int32_t* seqs;   /* int32[n_seqs][4], 16-byte aligned */
  int n_seqs, max_q_len, n_head, dk, dv;
  float scale;
  int dtype;
  /* optional (zero / NULL: absent).  k2: a key part of dk2 numbers per position shared by all heads, met by the LAST dk2 numbers
   * of each query head (dk counts the whole query head; k then holds dk - dk2 numbers per head).  sink: one logit per head (model
   * dtype) that joins the softmax denominator only.  gate: rows of ldg numbers; the output is multiplied by sigmoid(gate[row, h])
   * (gate_mode 1) or sigmoid(gate[row, h * dv + c]) (gate_mode 2). */
  const void* k2; int64_t ldk2; int dk2;
  const void* sink;
  const void* gate; int64_t ldg; int gate_mode;
} b200_latent_prefill_args;
int b200_latent_prefill(const b200_latent_prefill_args* args, b200_stream_t stream);
/* The same attention on the tensor cores for bf16 operands with dk = dv = head_size in {64, 128} (the kernel of b200_attn_prefill
 * over packed operands): leading dimensions multiples of 8 elements, q / k / v / seqs 16-byte aligned. */
int b200_attn_prefill_ragged(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, const int32_t* seqs,
                             int n_seqs, int max_q_len, void* y, int64_t ldy, int n_head, int head_size, float scale, b200_stream_t stream);
/* The same tiles for latent attention with a key part shared by the heads (bf16): q (rows, n_head * (head_size + dk2)), each head laid
 * out [head_size | dk2]; k, v (context rows, n_head * head_size); k2 (context rows, dk2); head_size and dk2 in {64, 128}; sink, gate and
 * gate_mode as in b200_latent_prefill_args (NULL / 0: absent). */
int b200_attn_prefill_shared(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, const void* k2, int64_t ldk2,
                             int dk2, const int32_t* seqs, int n_seqs, int max_q_len, void* y, int64_t ldy, int n_head, int head_size, float scale,
                             const void* sink, const void* gate, int64_t ldg, int gate_mode, b200_stream_t stream);
/* One query row per sequence over cached latents (slots, max_seq, r): sequence b reads positions 0 .. row_pos[b] of slot
 * row_slot[b] (its own latent already stored).  w_uk (n_head * dk, r) and w_uv (n_head * dv, r) are absorbed: no keys or
 * values are materialised.  n_split CTAs share each (sequence, head); the workspace holds their partial results. */
typedef struct b200_latent_decode_args {
  const void* q; const void* w_uk; const void* w_uv; const void* cache; void* out;
  int64_t ldq, ldo, slot_stride;
  const int32_t* row_slot; const int32_t* row_pos;
  int batch, n_head, dk, dv, r, max_seq, n_split;
  float scale;
  int dtype;
  void* workspace; size_t workspace_bytes;
  /* optional (zero / NULL: absent), as in b200_latent_prefill_args.  With dk2 > 0 a query head is [dk | dk2] numbers and a cache row
   * [r latent | dk2 shared key part]: slot_stride and the workspace count r + dk2 numbers per row. */
  int dk2;
  const void* sink;
  const void* gate; int64_t ldg; int gate_mode;
} b200_latent_decode_args;
size_t b200_latent_decode_workspace_bytes(int batch, int n_head, int r, int n_split);
int b200_latent_decode(const b200_latent_decode_args* args, b200_stream_t stream);
/* test knob: non-zero keeps bf16 decode on the any-size kernel instead of the tensor-core one; returns the previous setting */
int b200_latent_decode_tune(int force_any_size_kernel);

/* Router: s = sigmoid(W_router x), or softmax over all experts with B200_ROUTE_SOFTMAX; experts are chosen by s + correction among
 * the `keep` best of `n_group` equal groups of neighbours (group rank = sum of its two largest corrected scores, or the largest
 * with B200_ROUTE_GROUP_MAX); weights[t, k] = s of the chosen expert, not renormalised.  B200_ROUTE_TOPK_SOFTMAX: s is the raw logit,
 * the largest logits are chosen and the weights are a softmax among those `top` logits.  B200_ROUTE_BIAS: `correction` is a bias
 * added to the logit itself (it enters the scores) instead of a selection-only term. */
enum b200_route_flags { B200_ROUTE_SOFTMAX = 1, B200_ROUTE_GROUP_MAX = 2, B200_ROUTE_TOPK_SOFTMAX = 4, B200_ROUTE_BIAS = 8 };
int b200_moe_route(const void* x, const void* w_router, const void* correction, int32_t* ids, float* weights, int64_t tokens, int d,
                   int n_expert, int top, int n_group, int keep, int flags, int dtype, b200_stream_t stream);
/* counting sort of the (token, choice) pairs by expert: expert_off[E + 1], tile_off[E + 1] (64-row tiles), slot_token[tokens * top],
 * slot_of[tokens * top] */
int b200_moe_plan(const int32_t* ids, int64_t tokens, int top, int n_expert, int32_t* expert_off, int32_t* tile_off, int32_t* slot_token,
                  int32_t* slot_of, b200_stream_t stream);
/* c[row, :n] = act(a[row_src ? row_src[row] : row, :k] . w[e][:n, :k]^T) for the rows of every expert e; act = relu^2 or none */
int b200_moe_gemm(const void* a, int64_t lda, const int32_t* row_src, const void* w, void* c, int64_t ldc, const int32_t* expert_off,
                  const int32_t* tile_off, int64_t rows, int n_expert, int n, int k, int sqrelu, int dtype, b200_stream_t stream);
/* few tokens: hidden = relu(W_up[e] x)^2 per (token, choice) -- gated 1: silu(W_up[e][:ff] x) * (W_up[e][ff:] x) with 2 ff rows per
 * expert; gated 2: g sigmoid(alpha g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit) --,
 * out[t] = sum_k weights[t, k] * W_down[e_k] hidden[t, k] */
int b200_moe_gemv(const void* x, const int32_t* ids, const float* weights, const void* w_up, const void* w_down, void* hidden, void* out,
                  int64_t tokens, int top, int d, int ff, int gated, float limit, float alpha, int dtype, b200_stream_t stream);
int b200_moe_combine(const void* y, const int32_t* slot_of, const float* weights, void* out, int64_t tokens, int top, int d, int dtype,
                     b200_stream_t stream);

/* The tensor-core tiles of b200_attn_prefill for sequences that start in this step (every seqs[b] at position 0): bf16, dk = dv =
 * head_size in {64, 128}, grouped key-value heads, a sliding window (0: none) and per-head sink logits (NULL: none).  k and v are
 * the step's own rows (rows, n_kv_head * head_size). */
int b200_attn_prefill_window(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, const int32_t* seqs,
                             int n_seqs, int max_q_len, void* y, int64_t ldy, int n_head, int n_kv_head, int head_size, float scale,
                             int window, const void* sink, b200_stream_t stream);
/* The same with a distance bias (score -= r1[h] ln(1 + r2[h] (i - j)); both NULL: none) and a sigmoid output gate (gate_mode 0 none,
 * 1 gate[row, h], 2 gate[row, h * head_size + c]; rows ldg apart), all bf16. */
int b200_attn_prefill_window_ex(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, const int32_t* seqs,
                                int n_seqs, int max_q_len, void* y, int64_t ldy, int n_head, int n_kv_head, int head_size, float scale,
                                int window, const void* sink, const void* r1, const void* r2, const void* gate, int64_t ldg, int gate_mode,
                                b200_stream_t stream);

/* ---- sequence-state mechanisms: short convolutions, the gated delta rule, windowed attention over a ring -------------------
 * A step's rows are the new tokens of several sequences packed one after another; seqs[s] = {first row, rows, position of the
 * first row, state slot} (int32[n_seqs][4], 16-byte aligned) and row_seq[row] = s. */

/* x += norm(y) * post_w [+ extra]; act = dtype(norm(x) * pre_w), with y = y0 or the mean of norm(y0) * w0 and norm(y1) * w1;
 * norm(z) = z / sqrt(mean(z^2) + eps).  post_w NULL: y joins as it is; pre_w NULL: act is not written. */
typedef struct b200_sandwich_args {
  const void* y0; const void* w0; const void* y1; const void* w1;
  const void* post_w; const float* extra; const void* pre_w;
  float* x; void* act;
  int64_t rows; int d; float eps; int dtype;
} b200_sandwich_args;
int b200_sandwich_residual(const b200_sandwich_args* args, b200_stream_t stream);
/* in place; kind 0 exact gelu (erf), 1 tanh gelu, 2 silu, 3 relu^2 */
int b200_activation(void* x, int64_t n, int kind, int dtype, b200_stream_t stream);
/* out[r, c] = act(in[r, c]) * in[r, ff + c] for in (rows, 2 ff) */
int b200_glu(const void* in, void* out, int64_t rows, int ff, int kind, int dtype, b200_stream_t stream);
/* in place: xIELU with its two raw parameters params[0..1] (in `dtype`): z > 0: softplus(p) z^2 + z / 2, else (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 */
int b200_xielu(void* x, int64_t n, const void* params, int dtype, b200_stream_t stream);
/* in (rows, 2 ff) = [gate | up] -> out (rows, ff) = g sigmoid(alpha g) (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit) */
int b200_glu_clamped(const void* in, void* out, int64_t rows, int ff, float limit, float alpha, int dtype, b200_stream_t stream);
/* x += y0 * s0 + (y1 + y2) * s1 + extra + row_add (fp32 stream, in place; every term optional, a NULL scale is 1; s0, s1, row_add are
 * d numbers, extra fp32 rows); cast = dtype(x) (optional); act = dtype(tanh(alpha[0] * x) * nw + nb) (nw NULL: skipped) */
typedef struct b200_scaled_residual_args {
  const void* y0; const void* s0; const void* y1; const void* y2; const void* s1;
  const float* extra; const void* row_add;
  float* x; void* cast;
  const void* alpha; const void* nw; const void* nb; void* act;
  int64_t rows;
  int d, dtype;
} b200_scaled_residual_args;
int b200_scaled_residual(const b200_scaled_residual_args* args, b200_stream_t stream);

/* One group of heads of a short causal convolution (see b200_short_conv). */
typedef struct b200_conv_group {
  const void* w;            /* (heads * dim, taps), model dtype; the last column multiplies the current token */
  void* out;                /* (rows, heads * dim) with leading dimension ld_out; fp32 when out_f32, else model dtype */
  int64_t ld_out;
  const double* inv_freq;   /* rot_dims / 2 angular frequencies (post = 1) */
  int col0;                 /* first column of the group in the input rows and in the tail */
  int heads, dim;
  int act;                  /* 0 none, 1 silu */
  int post;                 /* 0 none, 1 rotate then x / sqrt(mean(x^2) + eps), 2 x / sqrt(sum(x^2) + eps) */
  int rot_dims;
  int out_f32;
  float rot_mscale;         /* multiplies cos and sin */
  float post_scale;         /* multiplies the result */
  float eps;
} b200_conv_group;
/* y[t, c] = sum_j w[c, j] * in[t - taps + 1 + j, c] per sequence (zeros before position 0; rows before the step from tail
 * (slots, taps - 1, tail_cols)), then act and post per head.  in (rows, >= tail_cols) with leading dimension ld_in. */
int b200_short_conv(const void* in, int64_t ld_in, const b200_conv_group* groups, int n_groups, int taps, const void* tail,
                    int64_t tail_slot_stride, int tail_cols, const int32_t* seqs, const int32_t* row_seq, int64_t rows, int dtype,
                    b200_stream_t stream);
/* tail[slot] <- the last taps - 1 input rows of every sequence after this step (call after b200_short_conv) */
int b200_conv_tail_update(const void* in, int64_t ld_in, void* tail, int64_t tail_slot_stride, int tail_cols, int taps, const int32_t* seqs,
                          int n_seqs, int dtype, b200_stream_t stream);

/* Gated delta rule over fp32 states, one dk x dv matrix per (slot, head): per token S *= g; u = beta (v - S^T k); S += k u^T;
 * o = S^T q, with beta = sigmoid(beta_in) and g = exp(-exp(a_log) * softplus(decay_in + dt_bias)); decay_in and dt_bias hold one
 * number per head, or per head and key channel with channel_decay.  q, k (rows, kv_heads * dk), v (rows, heads * dv) and out are
 * fp32; the raw projections and parameters are in the model dtype.  A sequence at position 0 starts from S = 0. */
typedef struct b200_delta_rule_args {
  const float* q; const float* k; const float* v;
  int64_t ldq, ldk, ldv;
  const void* beta_in; int64_t ld_beta;
  const void* decay_in; int64_t ld_decay;
  const void* a_log; const void* dt_bias;
  float* state; int64_t state_slot_stride;   /* floats per slot: heads * b200_delta_rule_state_floats(dk, dv) or more */
  float* out; int64_t ldo;
  const int32_t* seqs; int n_seqs;
  int heads, kv_heads, dk, dv, channel_decay, dtype;
  int max_rows;   /* the longest sequence's rows in this step (a hint for the launch shape; 0: unknown, treated as 1) */
} b200_delta_rule_args;
int64_t b200_delta_rule_state_floats(int dk, int dv);
int b200_delta_rule(const b200_delta_rule_args* args, b200_stream_t stream);
/* out[row, h, :] = dtype(o / sqrt(mean(o^2) + eps) * weight * gate(z)) per head; gate 1 silu, 2 sigmoid */
int b200_gated_rms_heads(const float* o, int64_t ldo, const void* z, int64_t ldz, const void* weight, void* out, int64_t ld_out, int64_t rows,
                         int heads, int dv, int gate, float eps, int dtype, b200_stream_t stream);

/* Sliding-window attention with a per-head sink logit in the softmax denominator (sink NULL: none).  Row at position i sees
 * positions i - window < j <= i: those of this step from k / v (rows, n_kv_head * dk | dv), older ones from the rings
 * (slots, ring, n_kv_head * dk | dv) where position p sits in row p % ring. */
typedef struct b200_window_attn_args {
  const void* q; const void* k; const void* v; void* out;
  int64_t ldq, ldk, ldv, ldo;
  const void* k_ring; const void* v_ring;
  const void* sink;
  const int32_t* seqs;
  int n_seqs, max_q_len, ring, n_head, n_kv_head, dk, dv, window;
  float scale;
  int dtype;
  const int32_t* row_seq;   /* given (with rows): the step's rows also enter the rings, as b200_ring_store does; NULL: rings untouched */
  int64_t rows;
  /* optional: score -= dist_r1[h] * ln(1 + dist_r2[h] * (i - j)) (both n_head numbers in `dtype`, or both NULL) */
  const void* dist_r1; const void* dist_r2;
  /* optional: the output is multiplied by sigmoid(gate[row, h]) (gate_mode 1) or sigmoid(gate[row, h * dv + c]) (gate_mode 2); rows ldg apart */
  const void* gate; int64_t ldg; int gate_mode;
} b200_window_attn_args;
int b200_window_attn(const b200_window_attn_args* args, b200_stream_t stream);
/* test knob: non-zero keeps single-row steps on the tiled kernel; returns the previous setting */
int b200_window_attn_tune(int force_tiled_kernel);
/* the step's rows among each sequence's last `ring` positions go to their ring rows (call after b200_window_attn) */
int b200_ring_store(const void* k, int64_t ldk, const void* v, int64_t ldv, void* k_ring, void* v_ring, int ring, int kcols, int vcols,
                    const int32_t* seqs, const int32_t* row_seq, int64_t rows, int dtype, b200_stream_t stream);


/* ---- grouped norms with an average over depth, per-head rotation, attention whose scores mix over the heads ------------------ */
/* x_out = x_in + gnorm(y) * post_w (fp32; y NULL: x_out = x_in); avg = sum_{j < m} depth_w[j] X_j with X_j = stack + j * stack_stride
 * for j < m - 1 and X_{m-1} = x_out (avg NULL: skipped); act = dtype(gnorm(avg or x_out) * pre_w) (pre_w NULL: skipped).  gnorm cuts a
 * row into `groups` equal consecutive pieces and divides each by its own sqrt(mean(piece^2) + eps).  y, weights and act are `dtype`. */
typedef struct b200_depth_residual_args {
  const void* y; const void* post_w;
  const float* x_in; float* x_out;
  const float* stack; int64_t stack_stride; const void* depth_w; float* avg;
  const void* pre_w; void* act;
  int64_t rows; int d, groups, m; float eps; int dtype;
} b200_depth_residual_args;
int b200_depth_residual(const b200_depth_residual_args* args, b200_stream_t stream);
/* One group of heads of b200_head_rope: head h of a row is `dim` numbers at in + row * ld_in + h * in_stride and goes to
 * out + out_rows[row] * ld_out + h * out_stride (out_rows NULL: the row itself; a row < 0 is skipped; in place allowed).  norm_w
 * (dim numbers, NULL: no norm) is the weight of an RMS norm over the head; dimensions [rot_off, rot_off + rot_dims) turn by
 * position * freq[i] (fp32), pair i = (2 i, 2 i + 1) when interleaved, else (i, i + rot_dims / 2), cos and sin times mag. */
typedef struct b200_head_rope_seg {
  const void* in; void* out; const void* norm_w; const float* freq; const int64_t* out_rows;
  int64_t ld_in, ld_out;
  int heads, dim, in_stride, out_stride, rot_off, rot_dims, interleaved;
  float mag;
} b200_head_rope_seg;
int b200_head_rope(const b200_head_rope_seg* segs, int n_segs, const int32_t* row_pos, int64_t rows, float eps, int dtype, b200_stream_t stream);
/* Causal attention over cached keys and values in which the heads' scores are mixed before the softmax:
 *   s_g(i, j) = scale * q_g(i) . k_{g / (n_head / n_kv_head)}(j);  s'_h = sum_g talk[h, g] s_g;  p_h = exp(s'_h) / (exp(sink_h) + sum_j exp(s'_h))
 * (talk NULL: no mixing; sink NULL: an ordinary softmax).  q (rows, n_head * dk); sequence s = seqs[s] (first row, rows, first position,
 * cache slot) reads positions 0 .. of its slot: key row p at k_cache + (slot * max_seq + p) * ldk, value row likewise (its own rows
 * already stored).  n_split CTAs share the keys of one query tile; the workspace holds their partial results. */
typedef struct b200_talk_attn_args {
  const void* q; int64_t ldq;
  const void* k_cache; int64_t ldk; const void* v_cache; int64_t ldv;
  const void* talk; const void* sink;
  void* out; int64_t ldo;
  const int32_t* seqs; int n_seqs, max_q_len;
  int64_t rows;
  int n_head, n_kv_head, dk, dv, max_seq, n_split;
  float scale; int dtype;
  void* workspace; size_t workspace_bytes;
} b200_talk_attn_args;
/* The same attention for bf16 prompts with dk = dv = head_size in {64, 128} and at most 64 heads, on the tensor-core prefill tiles, as
 * three launches over fp32 score planes: raw scores, the mixing in place, softmax with the sink and the value product.  sbuf holds
 * n_head planes of b200_attn_prefill_mixed_plane_floats(n_seqs, max_q_len, s_ld) floats each; s_ld is a multiple of 64 not below the
 * longest context.  Operands 16-byte aligned, leading dimensions multiples of 8. */
size_t b200_attn_prefill_mixed_plane_floats(int n_seqs, int max_q_len, int64_t s_ld);
int b200_attn_prefill_mixed(const void* q, int64_t ldq, const void* k_cache, int64_t ldk, const void* v_cache, int64_t ldv, const int32_t* seqs,
                            int n_seqs, int max_q_len, int max_seq, const void* talk, const void* sink, void* y, int64_t ldy, int n_head,
                            int n_kv_head, int head_size, float scale, float* sbuf, int64_t s_ld, b200_stream_t stream);
size_t b200_talk_attn_workspace_bytes(int64_t rows, int n_head, int dv, int n_split);
int b200_talk_attn(const b200_talk_attn_args* args, b200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200GPT_H */
