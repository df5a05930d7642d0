// Host entry points of the two attention forms (block attention over the paged
// KV cache for the denoising step, staircase attention over packed sequences
// for prefill), the merge of key-range parts, and the allocation-free variant
// of the paged entry.  The attention kernel itself (tcgen05 + TMA, one
// pipeline for both forms) lives in attention_tc.cu.
//
// Decode form: the key range of a request may be cut into nsplit parts that
// different CTAs process; partial (max, sum, O) triples go to a workspace and
// attn_combine_kernel merges them.
#include "mdb_common.cuh"

namespace mdb {

// Keys per key-range part of one request: an even share of its context rounded up to whole key tiles, but
// never fewer than 256 keys, so that a part count chosen for the longest admissible context does not cut a
// short one into single-tile parts (the trailing parts are then empty and cost one zero record each).
#ifndef MDB_ATTN_MIN_PART_KEYS
#define MDB_ATTN_MIN_PART_KEYS 256
#endif
constexpr int kAttnMinPartKeys = MDB_ATTN_MIN_PART_KEYS;
__host__ __device__ __forceinline__ int attn_part_keys(int ctx, int nsplit, int tile_keys) {
  if (ctx <= 0) return 0;
  const int share = ((ctx + nsplit - 1) / nsplit + tile_keys - 1) / tile_keys * tile_keys;
  return nsplit > 1 && share < kAttnMinPartKeys ? kAttnMinPartKeys : share;
}

struct AttnPagedArgs {
  const bf16* q;
  const bf16* k_cache;
  const bf16* v_cache;
  bf16* out;
  const int32_t* block_table;
  const int32_t* ctx_lens;
  float* part_o;   // [bs][nsplit][hq][block][128]
  float* part_ml;  // [bs][nsplit][hq][block][2]  (max in log2 units, sum)
  int table_stride, block, hq, hkv, num_pages, nsplit;
  float scale_log2;  // softmax_scale * log2(e)
};

// tcgen05/TMA form of the paged kernel (defined with the other tcgen05 kernels)
static bool attn_tc_supported(int block, int hq, int hkv, float softmax_scale);
static int attn_tc_launch(const AttnPagedArgs& a, int bs, cudaStream_t st);
struct AttnStairArgs;
static bool attn_stair_tc_supported(int hq, int hkv, int64_t q_stride, int64_t k_stride, int64_t v_stride);
static int attn_stair_tc_launch(const AttnStairArgs& a, int nseq, int max_seqlen, int64_t total_tokens, cudaStream_t st);

struct AttnStairArgs {
  const bf16* q;
  const bf16* k;
  const bf16* v;
  bf16* out;
  const int32_t* cu_seqlens;
  int64_t q_stride, k_stride, v_stride, out_stride;
  int hq, hkv, log2_stairs;
  float q_scale;  // log2(e) / sqrt(D)
};

// Merge the nsplit partials of one (request, head, token) row; one warp per row.
// Lanes first take one split each (running max and weighted sum across the
// warp), then every lane accumulates its 4 output columns over the splits
// with the weights broadcast by shuffle; the O loads are independent.
__device__ __forceinline__ void attn_combine_row(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                 bf16* __restrict__ out, int block, int hq, int nsplit,
                                                 int warp_global, int lane) {
  const int tok = warp_global % block;
  const int head = (warp_global / block) % hq;
  const int req = warp_global / (block * hq);
  const int64_t p0 = (static_cast<int64_t>(req) * nsplit * hq + head) * block + tok;   // split 0
  const int64_t pstride = static_cast<int64_t>(hq) * block;                             // between splits
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  // The O rows of the first eight parts are requested before anything depends on the (max, sum) records, so
  // that records and rows come back in one L2 round trip (every part's row is written, empty parts with zeros).
  float4 first[8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (i < nsplit) first[i] = *reinterpret_cast<const float4*>(part_o + (p0 + i * pstride) * kHeadDim + lane * 4);
  float mmax = -INFINITY;
  for (int s0 = 0; s0 < nsplit; s0 += 32) {   // running max over all splits
    const int s = s0 + lane;
    const float ms = s < nsplit ? part_ml[(p0 + s * pstride) * 2] : -INFINITY;
    mmax = fmaxf(mmax, ms);
  }
  mmax = warp_max(mmax);
  float lsum = 0.f;
  if (mmax != -INFINITY) {
    for (int s0 = 0; s0 < nsplit; s0 += 32) {
      const int s = s0 + lane;
      float w = 0.f, l = 0.f;
      if (s < nsplit) {
        const float2 ml = *reinterpret_cast<const float2*>(part_ml + (p0 + s * pstride) * 2);
        w = ml.x == -INFINITY ? 0.f : exp2f(ml.x - mmax);
        l = ml.y;
      }
      lsum += w * l;
      const int cnt = min(32, nsplit - s0);
      for (int j0 = 0; j0 < cnt; j0 += 8) {     // eight parts' rows in flight together, accumulated in part order
        float4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (j0 + i < cnt) {
            if (s0 + j0 == 0) v[i] = first[i];
            else if (__shfl_sync(0xffffffffu, w, j0 + i) != 0.f)   // empty parts are not fetched
              v[i] = *reinterpret_cast<const float4*>(part_o + (p0 + (s0 + j0 + i) * pstride) * kHeadDim + lane * 4);
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (j0 + i < cnt) {
            const float wj = __shfl_sync(0xffffffffu, w, j0 + i);
            if (wj != 0.f) {
              acc[0] += wj * v[i].x; acc[1] += wj * v[i].y; acc[2] += wj * v[i].z; acc[3] += wj * v[i].w;
            }
          }
        }
      }
    }
    lsum = warp_sum(lsum);
  }
  const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
  bf16* dst = out + ((static_cast<int64_t>(req) * block + tok) * hq + head) * kHeadDim + lane * 4;
  uint2 o;
  o.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
  o.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
  *reinterpret_cast<uint2*>(dst) = o;
}

__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    bf16* __restrict__ out, int bs, int block, int hq, int nsplit) {
  if (threadIdx.x == 0) trace_event(31, 0);
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) trace_event(31, 1);
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (warp_global >= bs * hq * block) return;
  attn_combine_row(part_o, part_ml, out, block, hq, nsplit, warp_global, threadIdx.x & 31);
  if (threadIdx.x == 0) trace_event(31, 2);
}

}  // namespace mdb

using namespace mdb;

extern "C" {

int64_t mdb_attn_paged_workspace_bytes(int bs, int block, int hq, int nsplit) {
  if (bs <= 0 || block <= 0 || hq <= 0 || nsplit <= 1) return 0;
  return static_cast<int64_t>(bs) * nsplit * hq * block * (kHeadDim + 2) * 4;
}

int mdb_attn_block_paged(const void* q, const void* k_cache, const void* v_cache, void* out,
                         const int32_t* block_table, int table_stride, const int32_t* ctx_lens, int bs, int block,
                         int hq, int hkv, int num_pages, float softmax_scale, int nsplit, void* workspace,
                         int64_t workspace_bytes, mdb_stream_t stream) {
  MDB_REQUIRE(bs >= 0 && block > 0 && hq > 0 && hkv > 0 && num_pages > 0 && table_stride > 0 && nsplit >= 1,
              MDB_ERR_ARG);
  if (bs == 0) return MDB_OK;
  MDB_REQUIRE(q && k_cache && v_cache && out && block_table && ctx_lens, MDB_ERR_ARG);
  MDB_REQUIRE(hq % hkv == 0, MDB_ERR_ARG);
  MDB_REQUIRE(bs <= 65535 && nsplit <= 1024, MDB_ERR_UNSUPPORTED);
  MDB_REQUIRE(mdb_aligned16(q) && mdb_aligned16(k_cache) && mdb_aligned16(v_cache) && mdb_aligned16(out) &&
                  mdb_aligned16(workspace),
              MDB_ERR_ALIGN);
  const int64_t need = mdb_attn_paged_workspace_bytes(bs, block, hq, nsplit);
  MDB_REQUIRE(need == 0 || (workspace != nullptr && workspace_bytes >= need), MDB_ERR_WORKSPACE);

  MDB_REQUIRE(attn_tc_supported(block, hq, hkv, softmax_scale), MDB_ERR_UNSUPPORTED);
  AttnPagedArgs a;
  a.q = static_cast<const bf16*>(q);
  a.k_cache = static_cast<const bf16*>(k_cache);
  a.v_cache = static_cast<const bf16*>(v_cache);
  a.out = static_cast<bf16*>(out);
  a.block_table = block_table;
  a.ctx_lens = ctx_lens;
  a.part_o = static_cast<float*>(workspace);
  a.part_ml = a.part_o ? a.part_o + static_cast<int64_t>(bs) * nsplit * hq * block * kHeadDim : nullptr;
  a.table_stride = table_stride;
  a.block = block;
  a.hq = hq;
  a.hkv = hkv;
  a.num_pages = num_pages;
  a.nsplit = nsplit;
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = attn_tc_launch(a, bs, st);
  if (rc != MDB_OK) return rc;
  if (nsplit > 1) {
    const int rows = bs * hq * block;
    const int threads = 256;
    const int blocks = (rows * 32 + threads - 1) / threads;
    rc = mdb_launch(attn_combine_kernel, dim3(blocks), dim3(threads), 0, st, a.part_o, a.part_ml, a.out, bs, block, hq,
                    nsplit);
  }
  return rc;
}

int mdb_attn_staircase_varlen(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                              int64_t v_stride, void* out, int64_t out_stride, const int32_t* cu_seqlens, int nseq,
                              int max_seqlen, int64_t total_tokens, int hq, int hkv, int stairs, mdb_stream_t stream) {
  MDB_REQUIRE(nseq >= 0 && max_seqlen >= 0 && hq > 0 && hkv > 0 && total_tokens >= 0, MDB_ERR_ARG);
  if (nseq == 0 || max_seqlen == 0) return MDB_OK;
  MDB_REQUIRE(q && k && v && out && cu_seqlens, MDB_ERR_ARG);
  MDB_REQUIRE(hq % hkv == 0, MDB_ERR_ARG);
  MDB_REQUIRE(stairs >= 1 && stairs <= 128 && (stairs & (stairs - 1)) == 0, MDB_ERR_UNSUPPORTED);
  MDB_REQUIRE(nseq <= 65535 && hq <= 65535, MDB_ERR_UNSUPPORTED);
  MDB_REQUIRE(q_stride >= static_cast<int64_t>(hq) * kHeadDim && out_stride >= static_cast<int64_t>(hq) * kHeadDim &&
                  k_stride >= static_cast<int64_t>(hkv) * kHeadDim && v_stride >= static_cast<int64_t>(hkv) * kHeadDim,
              MDB_ERR_ARG);
  MDB_REQUIRE(q_stride % 8 == 0 && k_stride % 8 == 0 && v_stride % 8 == 0 && out_stride % 8 == 0 &&
                  mdb_aligned16(q) && mdb_aligned16(k) && mdb_aligned16(v) && mdb_aligned16(out),
              MDB_ERR_ALIGN);
  MDB_REQUIRE(total_tokens > 0 && attn_stair_tc_supported(hq, hkv, q_stride, k_stride, v_stride), MDB_ERR_UNSUPPORTED);
  AttnStairArgs a;
  a.q = static_cast<const bf16*>(q);
  a.k = static_cast<const bf16*>(k);
  a.v = static_cast<const bf16*>(v);
  a.out = static_cast<bf16*>(out);
  a.cu_seqlens = cu_seqlens;
  a.q_stride = q_stride;
  a.k_stride = k_stride;
  a.v_stride = v_stride;
  a.out_stride = out_stride;
  a.hq = hq;
  a.hkv = hkv;
  int lg = 0;
  while ((1 << lg) < stairs) ++lg;
  a.log2_stairs = lg;
  a.q_scale = 1.0f / sqrtf(static_cast<float>(kHeadDim)) * 1.44269504f;
  return attn_stair_tc_launch(a, nseq, max_seqlen, total_tokens, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------
// Allocation-free variant of the paged block attention.
//
// Some hosts of this library cannot give it a workspace: an engine that has
// already handed every spare byte of the device to its KV-cache pool has no
// headroom left for a cudaMalloc, and a serving thread that must never stall
// cannot afford one either (cudaMalloc takes driver locks and may synchronise
// the device).  For them the split partials live in a fixed array inside the
// library image instead of a caller buffer.  The array is part of every
// device's copy of the module from load until the process exits.
//
// The array's name is only a host-side handle here: its device address is
// looked up once per device with cudaGetSymbolAddress (with that device
// current) on the first call made on that device, so make that first call
// outside any stream capture.  Nothing in the array has to start at zero: the
// attention kernel overwrites every (request, split, head, row) slot that
// the merge kernel then reads.  All calls on a device share the one array, so
// two calls that overlap on the GPU (different streams) race on it; keep
// them on one stream or order them with events.
constexpr int64_t kAttnStaticScratchBytes = 8ll << 20;   // 8 MiB, e.g. 16 splits x 16 heads x 32 rows for one request
static __device__ __align__(256) unsigned char g_attn_static_scratch[kAttnStaticScratchBytes];
static void* s_attn_static_scratch_ptr[64] = {};          // device address per device ordinal

int64_t mdb_attn_block_paged_noalloc_limit(void) { return kAttnStaticScratchBytes; }

int mdb_attn_block_paged_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                 const int32_t* block_table, int table_stride, const int32_t* ctx_lens, int bs,
                                 int block, int hq, int hkv, int num_pages, float softmax_scale, int nsplit,
                                 mdb_stream_t stream) {
  MDB_REQUIRE(bs >= 0 && block > 0 && hq > 0 && nsplit >= 1, MDB_ERR_ARG);
  const int64_t need = mdb_attn_paged_workspace_bytes(bs, block, hq, nsplit);
  MDB_REQUIRE(need <= kAttnStaticScratchBytes, MDB_ERR_STATIC_LIMIT);
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MDB_ERR_CUDA;
  if (s_attn_static_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_attn_static_scratch) != cudaSuccess || p == nullptr) return MDB_ERR_CUDA;
    s_attn_static_scratch_ptr[dev] = p;
  }
  return mdb_attn_block_paged(q, k_cache, v_cache, out, block_table, table_stride, ctx_lens, bs, block, hq, hkv,
                              num_pages, softmax_scale, nsplit, s_attn_static_scratch_ptr[dev], kAttnStaticScratchBytes,
                              stream);
}

}  // extern "C"
