/*
 * hqq_moe.h — C ABI of the B200 (sm_100a) quantized-expert library.
 *
 * Every entry point takes plain pointers and sizes, returns an int status
 * (HQM_OK = 0, negative = error; hqm_last_error() gives the message of the
 * calling thread's last failure), never throws, and — unless its comment says
 * otherwise — allocates no device memory: the caller owns every buffer and
 * passes the CUDA stream (a cudaStream_t cast to void*) the work is queued on.
 *
 * Activations are bf16 (uint16_t bit patterns here), row-major, contiguous.
 *
 * Weight layout (the one the reference keeps in memory after repack(),
 * src/custom_layers.py:41-47 and src/packing.py):
 *   W is (N, K) = (out_features, in_features); K is the contiguous axis and the
 *   packing runs along N: 4-bit uint8 (N/2, K), even row in the high nibble;
 *   2-bit uint8 (N/4, K), row n%4==0 in bits 7-6; 3-bit int32 (ceil(N/10), K),
 *   row n%10==i at bits 3*(9-i)+2..3*(9-i), rows past N zero.
 *   scale/zero: one pair per (n % G, k), G = N / group_size
 *   (src/triton_kernels.py:86-88,110-118); they are stored 8-bit (scale_q,
 *   zero_q: G*K bytes each) and decoded as (q - mz[c]) * ms[c] with
 *   c = (flat index) % (G*K / meta_group), ms/mz fp16 (src/custom_layers.py:62-66);
 *   scale and zero may use different meta_group sizes.
 */
#ifndef HQQ_MOE_H
#define HQQ_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HQM_OK 0
#define HQM_ERR_ARG (-1)      /* bad argument (null pointer, unsupported shape, misaligned buffer) */
#define HQM_ERR_CUDA (-2)     /* a CUDA runtime call failed */
#define HQM_ERR_SCRATCH (-3)  /* scratch buffer too small */
#define HQM_ERR_STATE (-4)    /* cache protocol violated (re-entrant request, unknown uid, full) */

/* One quantized linear layer: the tensors HQQLinearTritonSavable holds
 * (src/custom_layers.py:139-162: W_q, meta.scale_q, meta.meta_scale.{scale,zero},
 * meta.zero_q, meta.meta_zero.{scale,zero}) plus the non-tensor meta it reads in
 * forward_triton (src/custom_layers.py:68-84: shape, nbits, group_size). */
typedef struct hqm_weight {
    int32_t N, K;             /* meta['shape'] */
    int32_t nbits;            /* 2, 3 or 4 */
    int32_t group_size;       /* rows per quantisation group (axis 0) */
    int32_t meta_group;       /* group size of the 8-bit quantisation of scale (256) */
    int32_t meta_group_zero;  /* the same for zero; 0 = as meta_group.  (hqq's configs may differ between the two:
                                 the reference's notebook overrides the scale's only.)  Layers whose two sizes
                                 differ are computed by the shape-agnostic kernel, not the streaming ones. */
    const void* W_q;          /* packed codes, device pointer, 16-byte aligned */
    const uint8_t* scale_q;   /* G*K */
    const uint8_t* zero_q;    /* G*K */
    const uint16_t* ms_scale; /* fp16, G*K/meta_group: meta_scale.scale */
    const uint16_t* mz_scale; /* fp16: meta_scale.zero */
    const uint16_t* ms_zero;  /* fp16, G*K/meta_group_zero: meta_zero.scale */
    const uint16_t* mz_zero;  /* fp16: meta_zero.zero */
} hqm_weight;

const char* hqm_last_error(void);
int hqm_version(void);
/* Number of CUDA kernels this library has launched in the process so far (for benchmarks). */
int64_t hqm_launch_count(void);
/* 1 if a bounded wait inside a tensor-core GEMM launch ever ran out (that launch skipped its work),
 * 2 if hqm_attn_decode was given a position outside its cache, 3 if a streaming launch found the header of its
 * scratch buffer not zeroed (see hqm_scratch_init; its result is then incomplete), 4 if an expert-parallel
 * exchange gave up waiting for a peer, 0 otherwise, -1 on a CUDA error.  Reading a
 * non-zero value clears it.  Synchronises the device; meant for tests and start-up checks. */
int hqm_device_error(void);
/* No counterpart in the reference.  The streaming kernels and their reductions are launched so that a
 * kernel may become resident, set itself up and start requesting WEIGHT bytes while the kernel in front of
 * it on the stream is still finishing (programmatic dependent launch); activations, indices, outputs and
 * scratch are touched only after everything in front has completed.  The consequence for the caller: the
 * weight tensors of a call (W_q, scale_q, zero_q and the fp16 meta) must not be written by the work that
 * immediately precedes the call on the same stream; order such writes with an event, a copy or a
 * synchronisation, as a cache swap does.  hqm_set_overlap(0) switches to plain launches (so does
 * HQM_NO_OVERLAP=1 in the environment at load time), hqm_set_overlap(1) switches back; returns the previous
 * setting.  Process wide. */
int hqm_set_overlap(int on);

/* No counterpart in the reference.  Which single-row launches use the TMA-staged streaming kernel (tiled
 * cp.async.bulk.tensor copies of the packed tiles into per-warp stage rings, rows finished inside the kernel):
 * 0 = none, 1 = a linear that stands alone (hqm_linear, the default), 2 = also the multi-layer and table-driven
 * launches of hqm_expert_ffn / hqm_moe_decode / hqm_attn_decode / hqm_decode_layer.  HQM_TMA=0|1|2 in the
 * environment sets the initial value.  Returns the previous mode.  Process wide. */
int hqm_set_tma_mode(int mode);

/* ---- bit packing: src/packing.py --------------------------------------- */
/* pack_4bit_u8_common, packing.py:10-17.  codes (N, K) uint8 -> packed (N/2, K). */
int hqm_pack_4bit_u8(uint8_t* packed, const uint8_t* codes, int64_t N, int64_t K, void* stream);
/* unpack_4bit_u8_common, packing.py:19-27.  packed (rows, K) -> codes (2*rows, K). */
int hqm_unpack_4bit_u8(uint8_t* codes, const uint8_t* packed, int64_t rows, int64_t K, void* stream);
/* pack_2bit_u8_common, packing.py:36-41.  codes (N, K) -> packed (N/4, K). */
int hqm_pack_2bit_u8(uint8_t* packed, const uint8_t* codes, int64_t N, int64_t K, void* stream);
/* unpack_2bit_u8_common, packing.py:43-53.  packed (rows, K) -> codes (4*rows, K). */
int hqm_unpack_2bit_u8(uint8_t* codes, const uint8_t* packed, int64_t rows, int64_t K, void* stream);
/* pack_3bit_i32_common, packing.py:62-81.  codes (N, K) -> packed (ceil(N/10), K) int32. */
int hqm_pack_3bit_i32(int32_t* packed, const uint8_t* codes, int64_t N, int64_t K, void* stream);
/* unpack_3bit_i32_common, packing.py:83-97.  packed (rows, K) -> codes (10*rows, K). */
int hqm_unpack_3bit_i32(uint8_t* codes, const int32_t* packed, int64_t rows, int64_t K, void* stream);

/* ---- quantized linear: src/custom_layers.py:49-116, src/triton_kernels.py -- */
/* HQQLinearTritonSavable.dequantize, custom_layers.py:95-116: the full (N, K)
 * weight.  out_dtype: 0 = bf16, 1 = fp16, 2 = fp32. */
int hqm_dequantize(void* W_out, int out_dtype, const hqm_weight* w, void* stream);

/* No counterpart in the reference.  Every `scratch` buffer this library is given starts with
 * hqm_scratch_header_bytes() (64 KiB) of library state: arrival counters with which the CTAs of a streaming launch
 * that share a group of output rows decide which of them adds the parts up (so that no separate reduction launch
 * is needed).  The header must be zero the first time a buffer is used; hqm_scratch_init queues that memset on
 * `stream`.  Every call leaves the header zero again, so one initialisation per buffer is enough.  The sizes the
 * *_scratch_bytes functions return include the header.  Calls that share a scratch buffer must not overlap on
 * the GPU (they would also overwrite each other's partial sums). */
size_t hqm_scratch_header_bytes(void);
int hqm_scratch_init(void* scratch, void* stream);

/* Bytes of scratch hqm_linear needs for M rows of this layer (0 if none). */
size_t hqm_linear_scratch_bytes(int64_t M, const hqm_weight* w);

/* HQQLinearTritonSavable.forward / forward_triton (custom_layers.py:49-92) with the
 * kernels of triton_kernels.py:37-191 (4-bit), :225-380 (2-bit), :414-564 (3-bit)
 * and the per-call 8-bit scale/zero decode fused in:
 *   y[M, N] = x[M, K] . W_est^T (+ bias[N]),  fp32 accumulation, bf16 in/out.
 * bias may be NULL.  scratch may be NULL when hqm_linear_scratch_bytes() is 0.
 * Rows 1..16 take the weight-streaming kernels, 17 and more (5 and more for 3-bit layers) the tcgen05 kernels;
 * HQM_GEMM_TMA=0 in the environment at load time keeps the 2- and 4-bit many-row path on its first-generation
 * kernel (operand tiles filled by threads instead of TMA), HQM_FORCE_GENERIC=1 routes everything through the
 * shape-agnostic kernel. */
int hqm_linear(uint16_t* y, const uint16_t* x, int64_t M, const hqm_weight* w, const uint16_t* bias,
               void* scratch, size_t scratch_bytes, void* stream);

/* Same result as hqm_linear, for callers that cannot hand over a scratch buffer: code
 * running under CUDA stream capture (where allocating is not allowed), hosts that pass
 * raw pointers but own no device allocator, loops whose memory plan is frozen.  It has
 * no counterpart in the reference.  The partial sums go to a workspace built into the
 * library image (hqm_static_scratch_capacity() bytes, 2 MiB, held on every GPU that
 * loads the library until the process exits); the call allocates nothing.  A call that
 * would need more returns HQM_ERR_SCRATCH and says how much.  The first call on each
 * device looks up the workspace address (and, like hqm_linear, queries occupancy for a
 * new layer width), so make one call per device before starting a stream capture.  All
 * calls share the one workspace: calls that overlap on the GPU (different streams,
 * different threads) race; serialise them.  Nothing needs to be cleared between calls. */
size_t hqm_static_scratch_capacity(void);
int hqm_linear_static_scratch(uint16_t* y, const uint16_t* x, int64_t M, const hqm_weight* w, const uint16_t* bias,
                              void* stream);

/* ---- expert FFN: src/custom_layers.py:243-256 and :297-312 --------------- */
/* Bytes of scratch hqm_expert_ffn needs for M routed rows. */
size_t hqm_expert_ffn_scratch_bytes(int64_t M, const hqm_weight* w1, const hqm_weight* w2, const hqm_weight* w3);

/* MixtralBLockSparseTop2MLP_HQQ.forward (custom_layers.py:253-256) for the rows an
 * expert was routed, fused with the gather / routing-weight / index_add_ of
 * SparseMoeWrapper.forward (custom_layers.py:297-312):
 *   for i < M:  t = token_idx ? token_idx[i] : i
 *     h = w2( silu(w1 x[t]) * w3 x[t] )
 *     out[t] = (accumulate ? out[t] : 0) + (route_w ? route_w[i] : 1) * h
 * x and out are (tokens, hidden) bf16; token_idx int32[M] with distinct entries;
 * route_w float[M]. */
int hqm_expert_ffn(uint16_t* out, const uint16_t* x, int64_t M, const int32_t* token_idx, const float* route_w,
                   int accumulate, const hqm_weight* w1, const hqm_weight* w2, const hqm_weight* w3,
                   void* scratch, size_t scratch_bytes, void* stream);

/* ---- router: src/custom_layers.py:276-302 --------------------------------- */
/* Gate linear, fp32 softmax, top-2, renormalise (custom_layers.py:276-282) and the
 * per-expert token lists that one_hot/where build (custom_layers.py:290,297-302).
 *   x (M, K) bf16, gate_w (E, K) bf16, E <= 32.
 *   router_logits (M, E) bf16; topk_w (M, 2) float, rounded to bf16 as :282 casts;
 *   topk_idx (M, 2) int32; counts int32[E]; offsets int32[E+1];
 *   token_idx int32[2M] and token_w float[2M]: expert e owns
 *   [offsets[e], offsets[e+1]), tokens ascending. */
int hqm_router_top2(uint16_t* router_logits, float* topk_w, int32_t* topk_idx, int32_t* counts, int32_t* offsets,
                    int32_t* token_idx, float* token_w, const uint16_t* x, const uint16_t* gate_w, int64_t M,
                    int64_t K, int32_t E, void* stream);

/* No counterpart in the reference (its experts are Python modules picked on the host,
 * custom_layers.py:295-312).  The device-side expert table that hqm_moe_decode / hqm_decode_layer pick the
 * router's experts from: one 512-byte entry per weight, holding the descriptor and the three TMA tensor maps
 * (packed codes, scale bytes, zero bytes) the streaming kernel copies its tiles with.  hqm_expert_table_build
 * fills `host_out` (hqm_expert_table_bytes(n_weights) bytes, 64-byte aligned) on the HOST from n_weights
 * descriptors, ordered expert 0's w1, w2, w3, expert 1's w1, ...; the caller copies the bytes to device memory
 * (128-byte aligned) and passes that pointer as `table`.  The entries hold device addresses: rebuild the
 * table when a weight tensor moves.  Needs a CUDA driver (the tensor maps are encoded by it). */
size_t hqm_expert_table_bytes(int32_t n_weights);
int hqm_expert_table_build(void* host_out, const hqm_weight* weights, int32_t n_weights);

/* The whole of SparseMoeWrapper.forward (custom_layers.py:272-314) for ONE token when every expert is
 * resident on the device: router, then the two chosen experts' FFNs, weighted and summed into out (1, hidden).
 * Which experts run is decided on the device (the FFN kernels read the router's choice and fetch that
 * expert's entries from `table`), so nothing is copied back to the host and the call can be captured in a
 * CUDA graph.  table: the 3*E entries hqm_expert_table_build made, in DEVICE memory.
 * w1 / w2 / w3: host descriptors giving the (common) shapes and format.  router_logits: (1, E) bf16. */
size_t hqm_moe_decode_scratch_bytes(int32_t E, const hqm_weight* w1, const hqm_weight* w2, const hqm_weight* w3);
int hqm_moe_decode(uint16_t* out, uint16_t* router_logits, const uint16_t* x, const uint16_t* gate_w, int32_t E,
                   const void* table, const hqm_weight* w1, const hqm_weight* w2, const hqm_weight* w3,
                   void* scratch, size_t scratch_bytes, void* stream);

/* ---- the attention half of a decoder layer, one token ---------------------- */
/* The reference takes this step from the Hugging Face Mixtral decoder layer (build_model.py:166-241 builds the
 * model; the q/k/v/o projections inside it are HQQLinearTritonSavable, custom_layers.py:49-92).  It is offered
 * here, next to hqm_moe_decode, so that a whole decode step at batch 1 is a fixed sequence of launches:
 *     h += delta (when delta is given);  x = rmsnorm(h) * ln_in;
 *     q, k, v = projections of x;  rotate q and k by position *pos (rotate-half RoPE);
 *     k_cache[:, *pos] = k;  v_cache[:, *pos] = v;
 *     ctx = softmax(q K^T / sqrt(head_dim)) V over positions 0..*pos, n_heads / n_kv_heads query heads per
 *     key/value head;  h += o(ctx);  x_out = rmsnorm(h) * ln_post.
 * h (hidden) bf16 is the residual stream, updated in place; x_out (hidden) bf16 is the MoE block's input.
 * pos: one int32 in DEVICE memory (the caller advances it), so a captured graph can be replayed.
 * A position outside [0, max_len) writes nothing and makes hqm_device_error() return 2.
 * The four projections must share K-compatible streaming formats (2- or 4-bit); head_dim must be 128. */
typedef struct {
    hqm_weight q, k, v, o;
    const uint16_t* ln_in;    /* bf16 (hidden): input_layernorm.weight */
    const uint16_t* ln_post;  /* bf16 (hidden): post_attention_layernorm.weight */
    uint16_t* k_cache;        /* bf16 (n_kv_heads, max_len, head_dim) */
    uint16_t* v_cache;
    int32_t n_heads, n_kv_heads, head_dim, max_len;
    float rope_theta, rms_eps;
} hqm_attn_layer;
size_t hqm_attn_decode_scratch_bytes(const hqm_attn_layer* layer);
int hqm_attn_decode(uint16_t* h, uint16_t* x_out, const uint16_t* delta, const hqm_attn_layer* layer,
                    const int32_t* pos, void* scratch, size_t scratch_bytes, void* stream);
/* A whole decoder layer for one token, attention half and MoE block (hqm_attn_decode then hqm_moe_decode with
 * the residual adds and norms between them), as 8 launches: the steps between the quantized projections are
 * folded into their neighbours (RoPE / cache append into the attention kernel, the router into the
 * post-attention norm, the experts' weighted sum and the NEXT layer's input norm into one kernel).
 *   x   (hidden) bf16, in: rmsnorm(h) * this layer's input_layernorm weight (hqm_add_rmsnorm gives the first
 *       layer's); out: rmsnorm(updated h) * next_ln, i.e. the next layer's x (next_ln = the next layer's
 *       input_layernorm weight, or the model's final norm weight after the last layer).
 *   h   (hidden) bf16 residual stream, updated in place by both halves.
 *   router_logits (1, n_experts) bf16 out.  attn.ln_in is not used (x arrives normalised).
 *   table: the expert table in DEVICE memory as for hqm_moe_decode; w1 / w2 / w3 give the shapes. */
typedef struct {
    hqm_attn_layer attn;
    const uint16_t* gate_w;   /* bf16 (n_experts, hidden) */
    const void* table;
    hqm_weight w1, w2, w3;
    const uint16_t* next_ln;  /* bf16 (hidden) */
    int32_t n_experts, reserved;
} hqm_decoder_layer;
size_t hqm_decode_layer_scratch_bytes(const hqm_decoder_layer* layer);
int hqm_decode_layer(uint16_t* h, uint16_t* x, uint16_t* router_logits, const hqm_decoder_layer* layer,
                     const int32_t* pos, void* scratch, size_t scratch_bytes, void* stream);
/* No counterpart in the reference (which has no distributed code; the block being sharded is
 * SparseMoeWrapper.forward, custom_layers.py:272-314).  hqm_decode_layer for ONE RANK of an expert-parallel group:
 * attention, norms and router run replicated (every rank computes the same routing); the rank owns experts
 * [expert_lo, expert_lo + n_local) of the layer's n_experts and `layer->table` holds only those (3 * n_local
 * entries).  On the device the routed experts that the rank owns are packed into its launch slots (one slot when
 * it owns a single expert, else two); a slot without an expert streams nothing and contributes zeros.  The
 * residual stream h is updated by the attention half only, x is left untouched, and y_partial (hidden) receives
 * the rank's fp32 share of the MoE block's output: sum over its slots of bf16(weight * bf16(expert output)).
 * The caller adds the ranks' shares (an all-reduce on the same stream; every term is a bf16 value and at most two
 * are non-zero, so the fp32 sum is exact) and finishes the layer with hqm_add_f32_rmsnorm(h, y_sum, next_ln, x),
 * which gives bit for bit what hqm_decode_layer gives on one GPU.
 *
 * With `comm` set the exchange needs no collective library: the kernel that forms the rank's share stores it
 * straight into EVERY rank's exchange buffer over NVLink (plain peer stores, then one flag per 256 elements), and
 * hqm_ep_combine_add_rmsnorm waits for all ranks' flags, adds the shares in rank order and finishes the layer:
 * two launches between the experts and the next layer.  Each rank provides hqm_ep_exchange_bytes(world, hidden)
 * bytes of zeroed device memory that its peers can address (symmetric / IPC-mapped memory); shares[r] is rank r's
 * buffer as seen from this rank, flags[r] the same buffer + hqm_ep_exchange_flags_offset(); seq is one zeroed
 * uint32 in this rank's own memory.  All ranks must make the same sequence of exchanges.  Waits on a peer are
 * bounded (a fraction of a second); a flag that never arrives makes hqm_device_error() return 4. */
typedef struct hqm_ep_comm {
    int32_t rank, world;      /* world <= 8 */
    int32_t hidden, reserved;
    float* shares[8];
    uint32_t* flags[8];
    uint32_t* seq;
} hqm_ep_comm;
size_t hqm_ep_exchange_bytes(int32_t world, int32_t hidden);
size_t hqm_ep_exchange_flags_offset(int32_t world, int32_t hidden);
size_t hqm_decode_layer_ep_scratch_bytes(const hqm_decoder_layer* layer, int32_t n_local);
int hqm_decode_layer_ep(uint16_t* h, uint16_t* x, uint16_t* router_logits, float* y_partial, const hqm_ep_comm* comm,
                        const hqm_decoder_layer* layer, int32_t expert_lo, int32_t n_local, const int32_t* pos,
                        void* scratch, size_t scratch_bytes, void* stream);
int hqm_ep_combine_add_rmsnorm(uint16_t* h, const hqm_ep_comm* comm, const uint16_t* weight, uint16_t* x_out,
                               int32_t hidden, float eps, void* stream);
/* h = bf16(h + bf16(delta)) with delta in fp32; x_out = rmsnorm(h) * weight (see hqm_add_rmsnorm). */
int hqm_add_f32_rmsnorm(uint16_t* h, const float* delta, const uint16_t* weight, uint16_t* x_out, int32_t hidden,
                        float eps, void* stream);
/* h = bf16(h + delta) when delta is given; x_out = bf16(weight * bf16(h * rsqrt(mean(h^2) + eps))): the RMSNorm
 * of the Hugging Face decoder with the preceding residual add (used for the last layer's output and the final norm). */
int hqm_add_rmsnorm(uint16_t* h, const uint16_t* delta, const uint16_t* weight, uint16_t* x_out, int32_t hidden,
                    float eps, void* stream);
/* The same for `rows` rows at once (a prompt, a batch of sequences): h and delta (rows, hidden) bf16, x_out
 * (rows, hidden) bf16; delta may be NULL (then h is only read). */
int hqm_add_rmsnorm_rows(uint16_t* h, const uint16_t* delta, const uint16_t* weight, uint16_t* x_out, int64_t rows,
                         int32_t hidden, float eps, void* stream);
/* Rotary embedding and cache append for `tokens` tokens at once (modeling_mixtral.py apply_rotary_pos_emb and the
 * cache update of MixtralAttention.forward, with the arithmetic of hqm_attn_decode): q (tokens, n_heads, 128) bf16 is
 * rotated in place; k (tokens, n_kv_heads, 128) is rotated and, with v, written to row `pos` of the caches
 * (n_kv_heads, max_len, 128).  Token t has position base + t * pos_step, base = *pos_device (device memory) when
 * given, else pos0, and uses the cache batch_stride * t elements further on: a prompt has pos_step 1 and
 * batch_stride 0, a batch of sequences at one position pos_step 0 and batch_stride = the size of one cache. */
int hqm_rope_append_rows(uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* k_cache, uint16_t* v_cache,
                         int64_t tokens, int32_t n_heads, int32_t n_kv_heads, int32_t head_dim, int32_t max_len,
                         int64_t batch_stride, const int64_t* pos_device, int32_t pos0, int32_t pos_step, float rope_theta,
                         void* stream);

/* ---- expert residency: src/expert_cache.py -------------------------------- */
/* ExpertCache (expert_cache.py:55-201).  The handle owns the bookkeeping of
 * ExpertInfo / EvictionGroupInfo (expert_cache.py:12-52), a side copy stream and
 * the events that order it against the compute stream.  Slab memory stays with
 * the caller: `device_slabs` are main_size + buffer_size device buffers,
 * `host_slabs` one pinned buffer per registered expert (weights are immutable, so
 * an evicted expert is not copied back as expert_cache.py:189 does; its host copy
 * is still valid).  Passing NULL for both arrays gives a bookkeeping-only handle
 * (no CUDA calls), which is what the CPU tests drive. */
typedef struct hqm_cache hqm_cache;

int hqm_cache_create(hqm_cache** out, int32_t main_size, int32_t offload_size, int32_t buffer_size,
                     size_t slab_bytes, void* const* device_slabs, int32_t device_id);
void hqm_cache_destroy(hqm_cache* c);

/* add_expert_storage, expert_cache.py:93-118.  uid is any caller-chosen 64-bit key.
 * offload: 0 = device, 1 = host, -1 = device if room else host (None).
 * host_slab: this expert's pinned copy (may be NULL for a bookkeeping-only handle);
 * when the expert is placed on the device its bytes are copied there on `stream`.
 * *placed_offloaded receives 0/1.  HQM_ERR_STATE "Cache is full" when nothing fits. */
int hqm_cache_add(hqm_cache* c, int64_t uid, int32_t eviction_group, int32_t offload, const void* host_slab,
                  int32_t* placed_offloaded, void* stream);

/* load_experts, expert_cache.py:120-179, split into begin / next / end because a C
 * ABI has no generators.  begin: validates (distinct uids, one group, not
 * re-entrant), marks all as used, issues the first window of host->device copies
 * on the copy stream.  order_out receives the uids in the order they will be
 * yielded. */
int hqm_cache_begin(hqm_cache* c, const int64_t* uids, int32_t n, int32_t unordered, int64_t* order_out,
                    void* compute_stream);
/* Yields the next expert: *uid_out, and *slab_out = the device slab its bytes are
 * (or will be, in stream order) in.  The compute stream is made to wait for the
 * copy that fills it; the previous expert's compute is fenced so its slab can be
 * reused; one more copy is issued as expert_cache.py:171-175 does.  Returns 1 when
 * nothing is left (and then behaves as hqm_cache_end). */
int hqm_cache_next(hqm_cache* c, int64_t* uid_out, void** slab_out, int32_t* slot_out, void* compute_stream);
int hqm_cache_end(hqm_cache* c, void* compute_stream);

/* Speculative loading: the reference lists it as upcoming (README.md:24-27) and has no code for it.  Outside a
 * request, the offloaded ones among `uids` are brought onto the device as a miss would bring them (the group's
 * least recently used resident expert leaves; the copy runs on the side stream and is awaited when the expert is
 * used), without counting hits or misses and without touching experts that are resident already.  *issued_out =
 * copies started.  hqm_cache_prefetch_stats: copies started, guesses that were then asked for, guesses evicted
 * unused. */
int hqm_cache_prefetch(hqm_cache* c, const int64_t* uids, int32_t n, int32_t* issued_out);
int hqm_cache_prefetch_stats(hqm_cache* c, int64_t* issued, int64_t* used, int64_t* wasted);

/* hits / misses of a group (expert_cache.py:25-26) and copy counters. */
int hqm_cache_stats(hqm_cache* c, int32_t eviction_group, int64_t* hits, int64_t* misses, int64_t* h2d_bytes,
                    int64_t* swaps);
/* The group's resident uids, least recently used first; returns how many. */
int hqm_cache_resident(hqm_cache* c, int32_t eviction_group, int64_t* uids_out, int32_t cap);

#ifdef __cplusplus
}
#endif
#endif /* HQQ_MOE_H */
