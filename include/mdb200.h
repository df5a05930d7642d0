/*
 * libmdb200 -- C ABI of the B200 (sm_100a) block-diffusion decode kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (cudaStream_t passed as void*); nothing here names a torch type.  All
 * buffers are owned by the caller.  Calls are asynchronous on `stream`, do
 * not allocate and do not synchronise unless stated.  The return value is
 * MDB_OK or a negative MDB_ERR_* detected on the host before any launch.
 * Conditions only the device can see (a cache slot outside the pool, a
 * bounded wait that ran out) set a bit in a device status word instead of
 * trapping; read it with mdb_last_device_status().
 *
 * Paths in the comments are relative to the reference project root; NV/
 * abbreviates engines/nano_dvlm/nanovllm/.  bf16 means __nv_bfloat16.
 */
#ifndef MDB200_H
#define MDB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* mdb_stream_t; /* cudaStream_t */

enum {
  MDB_OK = 0,
  MDB_ERR_ARG = -1,         /* null pointer, non-positive size, inconsistent dims */
  MDB_ERR_ALIGN = -2,       /* pointer or stride not 16-byte aligned */
  MDB_ERR_UNSUPPORTED = -3, /* shape outside what the kernels are built for */
  MDB_ERR_CUDA = -4,        /* the launch itself was refused by the runtime */
  MDB_ERR_WORKSPACE = -5,   /* workspace smaller than *_workspace_bytes() */
  MDB_ERR_STATIC_LIMIT = -6 /* request needs more than the fixed scratch of an allocation-free entry point */
};

/* bits of the device status word */
enum {
  MDB_STATUS_BAD_SLOT = 1u,     /* slot_mapping entry outside [0, num_slots) and not -1: row skipped */
  MDB_STATUS_BAD_PAGE = 2u,     /* page-table entry outside [0, num_pages) (page 0 is read in its place) or a context
                                   longer than the page-table row can address (cut to the row): output rows invalid */
  MDB_STATUS_BAD_TOKEN = 4u,    /* token id outside the embedding table: row zeroed */
  MDB_STATUS_BAD_POSITION = 8u, /* position outside the rotary table: row left unrotated */
  MDB_STATUS_WAIT_TIMEOUT = 16u, /* a bounded wait on a peer flag or barrier expired */
  MDB_STATUS_LAYOUT = 32u        /* a kernel found its shared memory placed otherwise than it was built for and did nothing */
};

const char* mdb_strerror(int code);
int mdb_version(void);

/* Process-wide switches (no counterpart in the reference; for measurement and
 * fault isolation).  MDB_OPT_PDL: 1 = kernels are chained with programmatic
 * dependent launch (default), 0 = plain stream order.  MDB_OPT_GEMM_PAIR: GEMMs
 * of many rows on pairs of CTAs (tcgen05.mma.cta_group::2, tiles of 256 x 256):
 * 1 = from 2048 rows (default), 2 = from 256 rows, 0 = never.
 * MDB_OPT_WAIT_LIMIT_US: how long a wait inside a kernel (mbarrier, peer flag)
 * may last before it gives up and raises MDB_STATUS_WAIT_TIMEOUT, in
 * microseconds (default 2 000 000); written to the current device, blocking. */
enum { MDB_OPT_PDL = 1, MDB_OPT_GEMM_PAIR = 3, MDB_OPT_WAIT_LIMIT_US = 4 };
int mdb_set_option(int option, int value);
/* Measurement aid: registers a device buffer (uint64 count, then (kernel,
 * event, globaltimer ns) triples) that block 0 of the traced kernels appends
 * to; NULL switches tracing off.  The stamps exist only in a library built
 * with -DMDB_TRACE (MDB_TRACE=1 python mineru-diffusion_b200/build.py); in the
 * normal build the call registers the buffer and nothing is ever written to
 * it: even testing the buffer pointer in the kernels costs 7 % of a short step. */
int mdb_set_trace(void* buffer, int64_t bytes);
int mdb_get_option(int option);

/* Copies the status word of the current device to *out (host memory) after
 * synchronising the device; clear != 0 resets it.  Plays the part of the
 * reference's host asserts (NV/layers/attention.py:36-39). */
int mdb_last_device_status(unsigned int* out, int clear);

/* ---- paged KV write/commit --------------------------------------------- */

/* Replaces store_kvcache / store_kvcache_kernel (NV/layers/attention.py:10-40).
 * Row i of key/value (row_elems = Hkv*D bf16, row strides in elements) is
 * copied to k_cache/v_cache row slot_mapping[i]; slot -1 skips the row. */
int mdb_kv_commit(const void* key, int64_t key_stride, const void* value, int64_t value_stride, void* k_cache,
                  void* v_cache, const int32_t* slot_mapping, int n_tokens, int row_elems, int64_t num_slots,
                  mdb_stream_t stream);

/* ---- block attention over the paged cache (decode / denoise step) -------- */

/* Replaces flash_attn_with_kvcache(q, k_cache, v_cache, cache_seqlens,
 * block_table, softmax_scale, causal=False) as called at
 * NV/layers/sdar_attention.py:50-55.  q/out: [bs, block, hq, 128] bf16;
 * caches: [num_pages, 256, hkv, 128] bf16; block_table: [bs, table_stride]
 * int32 (-1 padded); ctx_lens: [bs] int32, 0 makes the request a no-op (its
 * output rows are zeroed).  Every query row sees keys [0, ctx).  The key range
 * of each request is cut into at most nsplit parts processed by different
 * CTAs (equal shares of its context, rounded up to whole key tiles and never
 * shorter than 256 keys, so a short context uses fewer parts than asked for);
 * nsplit > 1 needs the workspace. */
int64_t mdb_attn_paged_workspace_bytes(int bs, int block, int hq, int nsplit);
int mdb_attn_block_paged(const void* q, const void* k_cache, const void* v_cache, void* out,
                         const int32_t* block_table, int table_stride, const int32_t* ctx_lens, int bs, int block,
                         int hq, int hkv, int num_pages, float softmax_scale, int nsplit, void* workspace,
                         int64_t workspace_bytes, mdb_stream_t stream);

/* No counterpart in the reference.  Same operation and arguments as
 * mdb_attn_block_paged, but without a workspace argument: the split partials
 * go to a fixed 8 MiB array that lives inside the library (one per device,
 * held from load to exit), and the call allocates nothing.  It is meant for
 * hosts that cannot provide scratch memory, e.g. an engine whose KV-cache
 * pool has taken all remaining device memory, or a serving thread that must
 * not enter the allocator.  A request whose partials would not fit
 * (mdb_attn_paged_workspace_bytes(bs, block, hq, nsplit) above
 * mdb_attn_block_paged_noalloc_limit()) is refused with MDB_ERR_STATIC_LIMIT;
 * lower nsplit or bs.  The first call on each device resolves the array's
 * device address and should be made outside stream capture.  Calls share the
 * array: calls that overlap on the GPU race, so issue them on one stream. */
int64_t mdb_attn_block_paged_noalloc_limit(void);
int mdb_attn_block_paged_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                 const int32_t* block_table, int table_stride, const int32_t* ctx_lens, int bs,
                                 int block, int hq, int hkv, int num_pages, float softmax_scale, int nsplit,
                                 mdb_stream_t stream);

/* ---- staircase (block-causal, right-aligned) prefill attention ----------- */

/* Replaces sparse_attn_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k,
 * staircase_size) (NV/kernels/triton/attention/block_prefill_attention_v2.py:
 * 17-202, call site NV/layers/sdar_attention.py:39-47).  Packed sequences:
 * q/out rows of hq*128, k/v rows of hkv*128, row strides in elements;
 * cu_seqlens: [nseq+1] int32 (queries and keys share it: self-attention).
 * Query i of a T-token sequence sees keys j <= ((i+pad)/S+1)*S-1-pad with
 * pad = ceil(T/S)*S - T.  stairs must be a power of two in [1,128].
 * total_tokens = cu_seqlens[nseq] = the row count of q, k, v and out (the host
 * knows it; the TMA descriptors of the tcgen05 kernel are bounded by it). */
int mdb_attn_staircase_varlen(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                              int64_t v_stride, void* out, int64_t out_stride, const int32_t* cu_seqlens, int nseq,
                              int max_seqlen, int64_t total_tokens, int hq, int hkv, int stairs, mdb_stream_t stream);

/* ---- linear layers -------------------------------------------------------- */

/* In every entry of this section w is model data: with MDB_OPT_PDL on, a kernel
 * requests its first weight tiles while the preceding kernel of the stream may
 * still be running (weights are the only operand fetched that early), so w must
 * not be something a library call issued just before on the same stream writes.
 * Activations, outputs and workspaces carry the usual stream order. */

/* y[m,n] = x[m,k] * w[n,k]^T, bf16 in, fp32 accumulate, bf16 out: F.linear as
 * used by NV/layers/linear.py:72-73,153-154 and NV/layers/embed_head.py:67.
 * m <= 64 with n % 128 == 0 streams the weight once; everything else runs the
 * tcgen05 tile kernel (clusters of CTAs split k when the tiles are few, pairs
 * of CTAs share a tile from 2048 rows on); k % 64 == 0 and n % 8 == 0. */
int mdb_gemm_bf16(const void* x, int64_t ldx, const void* w, void* y, int64_t ldy, int m, int n, int k,
                  mdb_stream_t stream);

/* Same product for m <= 256 as a weight-streaming kernel that cuts k into
 * ksplit slices and writes fp32 partial sums partials[ksplit][m][n]; the
 * consumers below add the slices in index order, round to bf16 where F.linear
 * would, and apply the layer that follows.  (n % 128 == 0, k % 64 == 0, no
 * empty slice; the tensor-parallel form below takes m <= 64.) */
int mdb_gemm_pick_ksplit(int m, int n, int k); /* a ksplit that suits the kernel these shapes will run on */
int64_t mdb_gemm_splitk_workspace_bytes(int m, int n, int ksplit);
int mdb_gemm_splitk_partials(const void* x, int64_t ldx, const void* w, float* partials, int m, int n, int k,
                             int ksplit, mdb_stream_t stream);

/* gate_up projection fused with SiLU*mul (NV/models/sdar.py:109-111,
 * NV/layers/activation.py:12-15): w is [2*inter, k] with gate rows first;
 * act[m, inter] = bf16(silu_fp32(bf16(gate))) * bf16(up).  m <= 64 streams the
 * weight once (inter % 64 == 0, k % 64 == 0); larger m runs the tcgen05 tile
 * kernel (inter % 128 == 0, k % 64 == 0). */
int mdb_gemm_gateup_swiglu(const void* x, int64_t ldx, const void* w_gate_up, void* act, int64_t ld_act, int m,
                           int inter, int k, mdb_stream_t stream);

/* SiLU*mul on a materialised [m, 2*inter] bf16 matrix (SiluAndMul.forward, NV/layers/activation.py:12-15). */
int mdb_silu_mul(const void* gate_up, int64_t ld_in, void* act, int64_t ld_act, int m, int inter,
                 mdb_stream_t stream);

/* ---- fused reductions / element-wise layers -------------------------------- */

/* RMSNorm with fused residual add (NV/layers/layernorm.py:16-40).  The input
 * row is either x (bf16 [m,h]) or, when partials != NULL, the bf16-rounded
 * sum of nparts fp32 slices [nparts][m][h].  residual_in == NULL selects the
 * no-residual form (residual_out, if given, receives the input row). */
int mdb_add_rmsnorm(const void* x, const float* partials, int nparts, const void* residual_in, const void* weight,
                    float eps, void* y_out, void* residual_out, int m, int h, mdb_stream_t stream);

/* What follows qkv_proj in SDARAttention.forward (NV/models/sdar.py:73-82):
 * split q|k|v, per-head RMSNorm of q and k, NeoX rotary embedding from the
 * fp32 cos|sin table (NV/layers/rotary_embedding.py:6-48), then the KV store
 * of Attention.forward (NV/layers/sdar_attention.py:37-38).  Input row is
 * qkv (bf16 [m, (hq+2hkv)*128], row stride ld_qkv) or fp32 partials as above.
 * q_out [m, hq*128]; k_out/v_out [m, hkv*128] optional (prefill needs them
 * contiguous); slot_mapping optional (NULL: no cache write). */
int mdb_qknorm_rope_commit(const void* qkv, int64_t ld_qkv, const float* partials, int nparts,
                           const int64_t* positions, const float* rope_table, int max_pos, const void* q_norm_w,
                           const void* k_norm_w, float eps, const int32_t* slot_mapping, void* q_out, void* k_out,
                           void* v_out, void* k_cache, void* v_cache, int64_t num_slots, int m, int hq, int hkv,
                           mdb_stream_t stream);

/* qkv_proj and everything mdb_qknorm_rope_commit does, in one kernel for many
 * rows (prefill, batched decode): y = x w_qkv^T on the tcgen05 tile GEMM whose
 * epilogue rounds the projection to bf16, applies the per-head q/k RMSNorm and
 * the rotary embedding and stores q, k, v (NV/models/sdar.py:73-82,
 * NV/layers/sdar_attention.py:37-38) -- the [m, (hq+2hkv)*128] projection
 * never reaches memory.  x bf16 [m,k] (row stride ldx), w_qkv bf16
 * [(hq+2hkv)*128, k]; other arguments as mdb_qknorm_rope_commit.
 * MDB_ERR_UNSUPPORTED unless k % 64 == 0 and ldx % 8 == 0. */
int mdb_gemm_qkv_rope_commit(const void* x, int64_t ldx, const void* w_qkv, int m, int k, const int64_t* positions,
                             const float* rope_table, int max_pos, const void* q_norm_w, const void* k_norm_w,
                             float eps, const int32_t* slot_mapping, void* q_out, void* k_out, void* v_out,
                             void* k_cache, void* v_cache, int64_t num_slots, int hq, int hkv, mdb_stream_t stream);

/* Row gather: out[i,:] = table[ids[i],:] (F.embedding at
 * NV/layers/embed_head.py:38; also the last-block row pick of the LM head at
 * NV/layers/embed_head.py:63-66). */
int mdb_gather_rows(const void* table, int64_t num_rows, const int64_t* ids, void* out, int m, int h,
                    mdb_stream_t stream);

/* ---- LM head + sampler ------------------------------------------------------ */

/* Replaces ParallelLMHead.forward + Sampler.prepare (NV/layers/embed_head.py:
 * 61-72, NV/layers/sampler.py:11-22) without materialising logits: for each of
 * the m rows, logit_v = bf16(hidden . w[v]) / T, x0 = argmax_v(logit_v +
 * noise_v) (lowest index wins a tie), conf = softmax(logit)[x0].
 * temperatures: [m / block] fp32, one per request.  noise_mode 0: none,
 * 1: `noise` points to fp32 [m, vocab] Gumbel values, 2: counter-based Gumbel
 * noise from (seed, step, row, column) -- mdb_gumbel_noise() writes out the
 * same values.  step_dev, if not NULL, points to a uint32 in device memory
 * that is added to `step` when the kernel runs, so a captured graph can be
 * replayed with fresh noise.  m <= 64 streams the weight once; larger m runs
 * the tile GEMM with the sampler reduction in its epilogue (an explicit noise
 * tensor with many rows goes through bf16 logits in the workspace). */
int64_t mdb_lmhead_workspace_bytes(int m, int vocab);
int mdb_lmhead_sample(const void* hidden, int64_t ld_hidden, const void* w, int m, int vocab, int h,
                      const float* temperatures, int block, int noise_mode, const float* noise, uint32_t seed,
                      uint32_t step, const uint32_t* step_dev, void* workspace, int64_t workspace_bytes,
                      int32_t* x0_out, float* conf_out, mdb_stream_t stream);

/* Same scan over already materialised bf16 logits [m, vocab] (row stride ld);
 * a workspace of mdb_lmhead_workspace_bytes(m, vocab) always suffices. */
int mdb_logits_sample(const void* logits, int64_t ld, int m, int vocab, const float* temperatures, int block,
                      int noise_mode, const float* noise, uint32_t seed, uint32_t step, const uint32_t* step_dev,
                      void* workspace, int64_t workspace_bytes, int32_t* x0_out, float* conf_out,
                      mdb_stream_t stream);

int mdb_gumbel_noise(float* out, int m, int vocab, uint32_t seed, uint32_t step, mdb_stream_t stream);

/* The unmask rule of Sampler.forward (NV/layers/sampler.py:28-54) on device:
 * per request, masked positions whose confidence is > threshold are replaced
 * by x0; if fewer than the request's quota qualify, the quota most confident
 * masked positions are taken instead (all of them when fewer are left; the
 * lowest index wins a tie).  quota = 1 is the nano engine's rule; the HF twin
 * takes its quota from a per-block schedule
 * (mineru_diffusion/modeling_mineru_diffusion.py:518-532,617-623): pass it per
 * request in quotas [bs] int32 (device; NULL: `quota` for every request).
 * block_ids [bs, block] int64 is updated in place; transfer_out [bs, block]
 * uint8; count_out [bs] int32 = positions unmasked.  Requests with no masked
 * position are left untouched.  A quota of 0 (the schedule's entry when a block
 * has more steps than tokens) transfers only what passes the threshold.
 * status_out, if not NULL, is a device word that receives the device status
 * word as it stands when this kernel runs (the step's kernels before it have
 * finished), and the status word is cleared: the host reads the step's status
 * in the same copy as its results instead of synchronising for it. */
int mdb_unmask_decide(int64_t* block_ids, const int32_t* x0, const float* conf, int bs, int block, int64_t mask_id,
                      float threshold, int quota, const int32_t* quotas, uint8_t* transfer_out, int32_t* count_out,
                      uint32_t* status_out, mdb_stream_t stream);

/* ---- tensor-parallel pair (TP = 2) -------------------------------------------------- */

/* Replaces dist.all_reduce in RowParallelLinear.forward (NV/layers/linear.py:153-157),
 * the logits gather of ParallelLMHead (NV/layers/embed_head.py:68-71) and the
 * handle plumbing NCCL does for them.  Each rank holds half of the heads, MLP
 * columns and vocabulary tiles.  The o_proj / down_proj GEMM of a rank stores
 * its fp32 k-slices into its own slice buffer AND, over NVLink, into the
 * peer's (plain stores from the epilogue), then writes a sequence number into
 * its CTA's flag slot in the peer's memory.  The consumer (RMSNorm with
 * residual add) waits, bounded, for the peer's slots and sums rank 0's slices
 * then rank 1's, so both ranks obtain bit-identical rows.  Sequence number =
 * (*epoch) * 256 + tag; the host advances *epoch every step, tag (1..255) is
 * distinct per producing launch within a step. */

/* Device memory the peer may map: allocate, export a 64-byte handle, import the
 * peer's handle (in the other process), release/free at shutdown.  Called at
 * engine start only. */
int mdb_tp_alloc(int64_t bytes, void** out);
int mdb_tp_free(void* ptr);
int mdb_tp_export(void* ptr, void* handle_out64);
int mdb_tp_import(const void* handle64, void** peer_ptr_out);
int mdb_tp_release(void* peer_ptr);

/* mdb_gemm_splitk_partials whose slices also go to peer_partials (same layout,
 * peer memory) and that signals peer_flags[cta]; m <= 64, n % 128 == 0,
 * k % 64 == 0.  mdb_tp_grid_size gives the number of CTAs = flag slots used. */
int mdb_gemm_splitk_partials_tp(const void* x, int64_t ldx, const void* w, float* partials, float* peer_partials,
                                int m, int n, int k, int ksplit, uint32_t* peer_flags, uint32_t tag,
                                const uint32_t* epoch, mdb_stream_t stream);
int mdb_tp_grid_size(int m, int n, int k, int ksplit);

/* mdb_add_rmsnorm that first waits for wait_count flag slots written by the peer. */
int mdb_add_rmsnorm_tp(const void* x, const float* partials, int nparts, const void* residual_in, const void* weight,
                       float eps, void* y_out, void* residual_out, int m, int h, const uint32_t* wait_flags,
                       int wait_count, uint32_t tag, const uint32_t* epoch, mdb_stream_t stream);

/* The same exchange for steps of more than 64 rows (RowParallelLinear.forward +
 * dist.all_reduce, NV/layers/linear.py:153-157, on the tcgen05 tile GEMM):
 * mdb_gemm_bf16_tp stores every bf16 output tile into y and, with plain stores
 * over NVLink, into y_peer (the landing buffer in the peer's mdb_tp_alloc
 * memory, same leading dimension); each CTA then raises peer_flags[cta].
 * *grid_out = number of CTAs launched = flag slots the consumer has to wait
 * for (both ranks launch the same shape).  MDB_ERR_UNSUPPORTED unless m > 64
 * and the shape suits the tile kernel (k % 64 == 0, n % 8 == 0, ldy % 8 == 0).
 * mdb_add_rmsnorm_tp_rows waits for those slots and takes bf16(x + x_peer) as
 * its input row (x: this rank's output, x_peer: the local landing buffer the
 * peer wrote), which is what the all-reduce of two bf16 tensors yields. */
int mdb_gemm_bf16_tp(const void* x, int64_t ldx, const void* w, void* y, void* y_peer, int64_t ldy, int m, int n, int k,
                     uint32_t* peer_flags, uint32_t tag, const uint32_t* epoch, int* grid_out, mdb_stream_t stream);
int mdb_add_rmsnorm_tp_rows(const void* x, const void* x_peer, const void* residual_in, const void* weight, float eps,
                            void* y_out, void* residual_out, int m, int h, const uint32_t* wait_flags, int wait_count,
                            uint32_t tag, const uint32_t* epoch, mdb_stream_t stream);

/* mdb_lmhead_sample over the vocabulary tiles [tile_begin, tile_begin + tile_count)
 * (128 rows each) of the full weight; the per-tile records (20 bytes per step
 * row) are mirrored into the peer's workspace instead of gathering logits, and
 * the merge waits for the peer's records. */
int mdb_lmhead_sample_tp(const void* hidden, int64_t ld_hidden, const void* w, int m, int vocab, int h,
                         const float* temperatures, int block, int noise_mode, const float* noise, uint32_t seed,
                         uint32_t step, const uint32_t* step_dev, void* workspace, void* peer_workspace,
                         int64_t workspace_bytes, int tile_begin, int tile_count, uint32_t* peer_flags,
                         const uint32_t* wait_flags, int wait_count, uint32_t tag, const uint32_t* epoch,
                         int32_t* x0_out, float* conf_out, mdb_stream_t stream);
/* More than 64 rows: the same call runs the tcgen05 tile GEMM over the rank's
 * columns (tile_begin even; the shard ends on a multiple of 256 columns or at
 * the end of the vocabulary; no explicit noise tensor), one record per
 * 256-column tile, mirrored into the peer's workspace.  The workspace needs
 * mdb_lmhead_tp_workspace_bytes(m, vocab) bytes; the number of flag slots a
 * shard of `cols` columns raises (the peer's wait_count) is
 * mdb_lmhead_tp_slots(m, cols). */
int64_t mdb_lmhead_tp_workspace_bytes(int m, int vocab);
int mdb_lmhead_tp_slots(int m, int cols);

#ifdef __cplusplus
}
#endif
#endif /* MDB200_H */
