// Block attention for the denoising step (paged KV, every key visible) and
// staircase attention for prefill (packed sequences, right-aligned stairs).
//
// Both are flash-attention forward passes: a CTA of 4 warps owns 64 query rows
// (16 per warp), streams 64-key K/V tiles through a double-buffered shared
// memory ring filled with 16-byte cp.async, keeps S/P/O in registers and
// runs QK^T and PV on the tensor cores.  HBM traffic is K and V once; the
// arithmetic intensity of the decode form is block*hq/hkv flop per byte.
//
// Decode form: the hq/hkv query heads that share a KV head are packed with
// the block's rows into one row space (row = head_in_group*block + token) so
// that K/V of a request are read once per KV head.  The key range of a
// request is cut into nsplit parts (different CTAs); partial (max, sum, O)
// triples go to a workspace and a second kernel merges them.
#include "mdb_common.cuh"

namespace mdb {

constexpr int kAttnWarps = 4;
constexpr int kAttnRows = kAttnWarps * 16;  // query rows per CTA
constexpr int kAttnKeys = 64;               // keys per tile

// Keys per key-range part of one request: an even share of its context rounded up to whole key tiles, but
// never fewer than 256 keys, so that a part count chosen for the longest admissible context does not cut a
// short one into single-tile parts (the trailing parts are then empty and cost one zero record each).
__host__ __device__ __forceinline__ int attn_part_keys(int ctx, int nsplit, int tile_keys) {
  if (ctx <= 0) return 0;
  const int share = ((ctx + nsplit - 1) / nsplit + tile_keys - 1) / tile_keys * tile_keys;
  return nsplit > 1 && share < 256 ? 256 : share;
}
constexpr int kAttnTileBytes = kAttnKeys * kHeadDim * 2;
constexpr int kAttnSmemBytes = 2 /*stages*/ * 2 /*K,V*/ * kAttnTileBytes;  // 64 KB
constexpr int64_t kAttnTcMinTiles = 0;       // 128-key tiles (upper bound) from which the tcgen05 kernel is chosen: measured no slower at any size

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

// Issue the cp.async copies of one 64-key tile.  row_ptr(r) is the global
// address of key row r of the tile (nullptr: zero-fill).
template <typename RowPtr>
__device__ __forceinline__ void load_tile_async(uint32_t smem_tile, RowPtr row_ptr) {
  const int tid = threadIdx.x;
  const int chunk = tid & 15;
#pragma unroll
  for (int i = 0; i < kAttnKeys / 8; ++i) {
    const int row = (tid >> 4) + 8 * i;
    const bf16* src = row_ptr(row);
    const uint32_t dst = smem_tile + row * 256 + (swz_chunk(row, chunk) << 4);
    // the source address must stay valid even for a pure zero fill
    cp_async16(dst, src != nullptr ? static_cast<const void*>(src + chunk * 8) : static_cast<const void*>(&g_device_status),
               src != nullptr ? 16 : 0);
  }
}

// One 64-key step for a warp: S = Q K^T, mask, online softmax, O += P V.
// `score_scale` multiplies raw scores inside exp2 (decode form); the staircase
// form passes 1 because its Q is pre-scaled.  `limit0/limit1` are the last
// visible key index (inclusive) of rows g and g+8.
__device__ __forceinline__ void attn_tile_step(const uint32_t (&qf)[8][4], uint32_t k_tile, uint32_t v_tile,
                                               int key0, int limit0, int limit1, float score_scale, float (&o)[16][4],
                                               float (&m)[2], float (&l)[2]) {
  const int lane = threadIdx.x & 31;
  const int t = lane & 3;
  const int mat = lane >> 3, r8 = lane & 7;

  float s[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;

#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {      // 16 head-dim columns per step
#pragma unroll
    for (int jp = 0; jp < 4; ++jp) {    // two 8-key tiles per ldmatrix.x4
      const int row = 16 * jp + (mat >> 1) * 8 + r8;
      const int chunk = 2 * ks + (mat & 1);
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4(b0, b1, b2, b3, k_tile + row * 256 + (swz_chunk(row, chunk) << 4));
      mma_bf16_16816(s[2 * jp], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
      mma_bf16_16816(s[2 * jp + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
    }
  }

  // mask + row max
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int key = key0 + 8 * j + 2 * t;
    if (key > limit0) s[j][0] = -INFINITY;
    if (key + 1 > limit0) s[j][1] = -INFINITY;
    if (key > limit1) s[j][2] = -INFINITY;
    if (key + 1 > limit1) s[j][3] = -INFINITY;
    mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
    mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));

  const float mn0 = fmaxf(m[0], mx0 * score_scale);
  const float mn1 = fmaxf(m[1], mx1 * score_scale);
  // a row with nothing visible yet keeps max = -inf; use 0 as the exponent base
  const float base0 = (mn0 == -INFINITY) ? 0.f : mn0;
  const float base1 = (mn1 == -INFINITY) ? 0.f : mn1;
  const float alpha0 = exp2f(m[0] - base0);
  const float alpha1 = exp2f(m[1] - base1);
  m[0] = mn0;
  m[1] = mn1;

  float sum0 = 0.f, sum1 = 0.f;
  uint32_t pf[8][2];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float p0 = exp2f(fmaf(s[j][0], score_scale, -base0));
    const float p1 = exp2f(fmaf(s[j][1], score_scale, -base0));
    const float p2 = exp2f(fmaf(s[j][2], score_scale, -base1));
    const float p3 = exp2f(fmaf(s[j][3], score_scale, -base1));
    sum0 += p0 + p1;
    sum1 += p2 + p3;
    pf[j][0] = pack_bf16x2(p0, p1);
    pf[j][1] = pack_bf16x2(p2, p3);
  }
  l[0] = l[0] * alpha0 + sum0;
  l[1] = l[1] * alpha1 + sum1;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    o[j][0] *= alpha0; o[j][1] *= alpha0;
    o[j][2] *= alpha1; o[j][3] *= alpha1;
  }

#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {      // 16 keys per step
#pragma unroll
    for (int jp = 0; jp < 8; ++jp) {    // two 8-column tiles of the head dim
      const int row = 16 * kk + (mat & 1) * 8 + r8;
      const int chunk = 2 * jp + (mat >> 1);
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(b0, b1, b2, b3, v_tile + row * 256 + (swz_chunk(row, chunk) << 4));
      mma_bf16_16816(o[2 * jp], pf[2 * kk][0], pf[2 * kk][1], pf[2 * kk + 1][0], pf[2 * kk + 1][1], b0, b1);
      mma_bf16_16816(o[2 * jp + 1], pf[2 * kk][0], pf[2 * kk][1], pf[2 * kk + 1][0], pf[2 * kk + 1][1], b2, b3);
    }
  }
}

// ---------------------------------------------------------------------------
// decode form over the paged cache
// ---------------------------------------------------------------------------
// 128 threads synchronise either as a whole CTA or, inside the fused step kernel where two more warps
// do other work, on named barrier 1.
template <bool NAMED>
__device__ __forceinline__ void attn_sync() {
  if (NAMED) asm volatile("bar.sync 1, 128;" ::: "memory");
  else __syncthreads();
}

// One work item of the decode form: (request, KV head, 64-row block of the packed query rows, key-range split).
template <bool NAMED>
__device__ __forceinline__ void attn_paged_item(const AttnPagedArgs& a, uint32_t smem, int split, int kvh, int rb,
                                                int req) {
  const int group = a.hq / a.hkv;
  const int rows_total = group * a.block;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  const int ctx = a.ctx_lens[req];
  // equal key ranges per split, rounded to whole tiles
  const int chunk = attn_part_keys(ctx, a.nsplit, kAttnKeys);
  const int kbeg = split * chunk;
  const int kend = min(ctx, kbeg + chunk);
  const int ntiles = kend > kbeg ? (kend - kbeg + kAttnKeys - 1) / kAttnKeys : 0;

  // rows g and g+8 of this warp's 16-row tile, in the packed (head, token) space
  const int R0 = rb * kAttnRows + warp * 16 + g;
  const int R1 = R0 + 8;
  const bool valid0 = R0 < rows_total, valid1 = R1 < rows_total;
  const int head0 = kvh * group + (valid0 ? R0 / a.block : 0), tok0 = valid0 ? R0 % a.block : 0;
  const int head1 = kvh * group + (valid1 ? R1 / a.block : 0), tok1 = valid1 ? R1 % a.block : 0;
  const int64_t qoff0 = ((static_cast<int64_t>(req) * a.block + tok0) * a.hq + head0) * kHeadDim;
  const int64_t qoff1 = ((static_cast<int64_t>(req) * a.block + tok1) * a.hq + head1) * kHeadDim;

  uint32_t qf[8][4];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const int d = 16 * ks + 2 * t;
    qf[ks][0] = valid0 ? *reinterpret_cast<const uint32_t*>(a.q + qoff0 + d) : 0u;
    qf[ks][1] = valid1 ? *reinterpret_cast<const uint32_t*>(a.q + qoff1 + d) : 0u;
    qf[ks][2] = valid0 ? *reinterpret_cast<const uint32_t*>(a.q + qoff0 + d + 8) : 0u;
    qf[ks][3] = valid1 ? *reinterpret_cast<const uint32_t*>(a.q + qoff1 + d + 8) : 0u;
  }

  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY};
  float l[2] = {0.f, 0.f};

  const int row_elems = a.hkv * kHeadDim;
  auto issue = [&](int tile, int stage) {
    const int key0 = kbeg + tile * kAttnKeys;
    const int page_idx = key0 / kPage;
    int page = a.block_table[static_cast<int64_t>(req) * a.table_stride + page_idx];
    if (page < 0 || page >= a.num_pages) {
      if (threadIdx.x == 0) report_status(MDB_STATUS_BAD_PAGE);
      page = -1;
    }
    const int64_t base = page < 0 ? 0 : (static_cast<int64_t>(page) * kPage + (key0 % kPage)) * row_elems + kvh * kHeadDim;
    const int nvalid = page < 0 ? 0 : min(kAttnKeys, kend - key0);
    const uint32_t kt = smem + stage * 2 * kAttnTileBytes;
    const uint32_t vt = kt + kAttnTileBytes;
    load_tile_async(kt, [&](int r) { return r < nvalid ? a.k_cache + base + static_cast<int64_t>(r) * row_elems : nullptr; });
    load_tile_async(vt, [&](int r) { return r < nvalid ? a.v_cache + base + static_cast<int64_t>(r) * row_elems : nullptr; });
    cp_async_commit();
  };

  if (ntiles > 0) issue(0, 0);
  for (int it = 0; it < ntiles; ++it) {
    if (it + 1 < ntiles) {
      issue(it + 1, (it + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    attn_sync<NAMED>();
    const uint32_t kt = smem + (it & 1) * 2 * kAttnTileBytes;
    const int key0 = kbeg + it * kAttnKeys;
    attn_tile_step(qf, kt, kt + kAttnTileBytes, key0, kend - 1, kend - 1, a.scale_log2, o, m, l);
    attn_sync<NAMED>();
  }

  // quad-reduce the row sums
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);

  if (a.nsplit == 1) {
    const float inv0 = l[0] > 0.f ? 1.0f / l[0] : 0.f;
    const float inv1 = l[1] > 0.f ? 1.0f / l[1] : 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int d = 8 * j + 2 * t;
      if (valid0) *reinterpret_cast<uint32_t*>(a.out + qoff0 + d) = pack_bf16x2(o[j][0] * inv0, o[j][1] * inv0);
      if (valid1) *reinterpret_cast<uint32_t*>(a.out + qoff1 + d) = pack_bf16x2(o[j][2] * inv1, o[j][3] * inv1);
    }
    return;
  }
  // partials: [req][split][head][token]
  const int64_t p0 = ((static_cast<int64_t>(req) * a.nsplit + split) * a.hq + head0) * a.block + tok0;
  const int64_t p1 = ((static_cast<int64_t>(req) * a.nsplit + split) * a.hq + head1) * a.block + tok1;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int d = 8 * j + 2 * t;
    if (valid0) *reinterpret_cast<float2*>(a.part_o + p0 * kHeadDim + d) = make_float2(o[j][0], o[j][1]);
    if (valid1) *reinterpret_cast<float2*>(a.part_o + p1 * kHeadDim + d) = make_float2(o[j][2], o[j][3]);
  }
  if (t == 0) {
    if (valid0) *reinterpret_cast<float2*>(a.part_ml + p0 * 2) = make_float2(m[0], l[0]);
    if (valid1) *reinterpret_cast<float2*>(a.part_ml + p1 * 2) = make_float2(m[1], l[1]);
  }
}

__global__ void __launch_bounds__(kAttnWarps * 32)
attn_block_paged_kernel(const AttnPagedArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int group = a.hq / a.hkv;
  const int row_blocks = (group * a.block + kAttnRows - 1) / kAttnRows;
  attn_paged_item<false>(a, smem_u32(smem_raw), blockIdx.x, blockIdx.y / row_blocks, blockIdx.y % row_blocks,
                         blockIdx.z);
}

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

// ---------------------------------------------------------------------------
// staircase form over packed sequences
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kAttnWarps * 32)
attn_staircase_kernel(const AttnStairArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const uint32_t smem = smem_u32(smem_raw);
  const int seq = blockIdx.z;
  const int head = blockIdx.y;
  const int seq_start = a.cu_seqlens[seq];
  const int T = a.cu_seqlens[seq + 1] - seq_start;
  // heavy (late) query tiles first
  const int m0 = (gridDim.x - 1 - blockIdx.x) * kAttnRows;
  if (m0 >= T) return;
  const int kvh = head / (a.hq / a.hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  const int S = 1 << a.log2_stairs;
  const int pad = ((T + S - 1) >> a.log2_stairs << a.log2_stairs) - T;
  const int i0 = m0 + warp * 16 + g, i1 = i0 + 8;
  const bool valid0 = i0 < T, valid1 = i1 < T;
  // last visible key of each row (rows past the end see nothing)
  const int limit0 = valid0 ? min(T - 1, ((((i0 + pad) >> a.log2_stairs) + 1) << a.log2_stairs) - 1 - pad) : -1;
  const int limit1 = valid1 ? min(T - 1, ((((i1 + pad) >> a.log2_stairs) + 1) << a.log2_stairs) - 1 - pad) : -1;
  const int last_row = min(m0 + kAttnRows, T) - 1;
  const int end_n = min(T, ((((last_row + pad) >> a.log2_stairs) + 1) << a.log2_stairs) - pad);
  const int ntiles = (end_n + kAttnKeys - 1) / kAttnKeys;

  const bf16* q0 = a.q + static_cast<int64_t>(seq_start + (valid0 ? i0 : 0)) * a.q_stride + head * kHeadDim;
  const bf16* q1 = a.q + static_cast<int64_t>(seq_start + (valid1 ? i1 : 0)) * a.q_stride + head * kHeadDim;
  uint32_t qf[8][4];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const int d = 16 * ks + 2 * t;
    uint32_t raw[4];
    raw[0] = valid0 ? *reinterpret_cast<const uint32_t*>(q0 + d) : 0u;
    raw[1] = valid1 ? *reinterpret_cast<const uint32_t*>(q1 + d) : 0u;
    raw[2] = valid0 ? *reinterpret_cast<const uint32_t*>(q0 + d + 8) : 0u;
    raw[3] = valid1 ? *reinterpret_cast<const uint32_t*>(q1 + d + 8) : 0u;
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      // q is scaled by log2(e)/sqrt(D) and rounded to bf16 before the product
      const float2 f = unpack_bf16x2(raw[x]);
      qf[ks][x] = pack_bf16x2(f.x * a.q_scale, f.y * a.q_scale);
    }
  }

  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY};
  float l[2] = {0.f, 0.f};

  auto issue = [&](int tile, int stage) {
    const int key0 = tile * kAttnKeys;
    const int nvalid = min(kAttnKeys, T - key0);
    const bf16* kb = a.k + static_cast<int64_t>(seq_start + key0) * a.k_stride + kvh * kHeadDim;
    const bf16* vb = a.v + static_cast<int64_t>(seq_start + key0) * a.v_stride + kvh * kHeadDim;
    const uint32_t kt = smem + stage * 2 * kAttnTileBytes;
    const uint32_t vt = kt + kAttnTileBytes;
    load_tile_async(kt, [&](int r) { return r < nvalid ? kb + static_cast<int64_t>(r) * a.k_stride : nullptr; });
    load_tile_async(vt, [&](int r) { return r < nvalid ? vb + static_cast<int64_t>(r) * a.v_stride : nullptr; });
    cp_async_commit();
  };

  if (ntiles > 0) issue(0, 0);
  for (int it = 0; it < ntiles; ++it) {
    if (it + 1 < ntiles) {
      issue(it + 1, (it + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t kt = smem + (it & 1) * 2 * kAttnTileBytes;
    attn_tile_step(qf, kt, kt + kAttnTileBytes, it * kAttnKeys, limit0, limit1, 1.0f, o, m, l);
    __syncthreads();
  }

  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
  const float inv0 = l[0] > 0.f ? 1.0f / l[0] : 0.f;
  const float inv1 = l[1] > 0.f ? 1.0f / l[1] : 0.f;
  bf16* o0 = a.out + static_cast<int64_t>(seq_start + i0) * a.out_stride + head * kHeadDim;
  bf16* o1 = a.out + static_cast<int64_t>(seq_start + i1) * a.out_stride + head * kHeadDim;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int d = 8 * j + 2 * t;
    if (valid0) *reinterpret_cast<uint32_t*>(o0 + d) = pack_bf16x2(o[j][0] * inv0, o[j][1] * inv0);
    if (valid1) *reinterpret_cast<uint32_t*>(o1 + d) = pack_bf16x2(o[j][2] * inv1, o[j][3] * inv1);
  }
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

  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_block_paged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmemBytes) !=
        cudaSuccess)
      return MDB_ERR_CUDA;
    attr_set = true;
  }
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
  const int rows_total = hq / hkv * block;
  const int row_blocks = (rows_total + kAttnRows - 1) / kAttnRows;
  dim3 grid(nsplit, hkv * row_blocks, bs);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The tensor-core pipeline pays off once there are enough 128-key tiles to keep every SM streaming;
  // the context lengths live on the device, so the page-table width stands in for them.
  const int64_t tiles_bound = static_cast<int64_t>(bs) * hkv * table_stride * (kPage / 128);
  const bool want_tc = g_opt_attn_kernel == 2 || (g_opt_attn_kernel == 0 && tiles_bound >= kAttnTcMinTiles);
  int rc;
  if (want_tc && attn_tc_supported(block, hq, hkv, softmax_scale))
    rc = attn_tc_launch(a, bs, st);
  else
    rc = mdb_launch(attn_block_paged_kernel, grid, dim3(kAttnWarps * 32), kAttnSmemBytes, st, a);
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
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_staircase_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmemBytes) !=
        cudaSuccess)
      return MDB_ERR_CUDA;
    attr_set = true;
  }
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
  if (g_opt_attn_kernel != 1 && total_tokens > 0 && attn_stair_tc_supported(hq, hkv, q_stride, k_stride, v_stride))
    return attn_stair_tc_launch(a, nseq, max_seqlen, total_tokens, static_cast<cudaStream_t>(stream));
  dim3 grid((max_seqlen + kAttnRows - 1) / kAttnRows, hq, nseq);
  return mdb_launch(attn_staircase_kernel, grid, dim3(kAttnWarps * 32), kAttnSmemBytes,
                    static_cast<cudaStream_t>(stream), a);
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
