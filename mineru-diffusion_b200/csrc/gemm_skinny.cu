// Weight-streaming linear layers for a denoising step of at most 64 rows.
//
// With m <= 64 every projection is HBM-bound: each weight byte is read once and
// used for m multiply-adds.  The kernel therefore streams W with independent
// 16-byte loads straight into registers (no shared-memory staging: nothing is
// reused across warps) and feeds them to the tensor cores as the B operand of
// m16n8k16, the activations being the A operand.  Inside one MMA the k index is
// only a summation index, so each lane may take 8 *contiguous* k values of its
// weight row (one 16-byte load) and split them over two MMAs as long as the
// activation fragment uses the same assignment; this removes ldmatrix and
// shared memory from the weight path altogether.
//
// A CTA owns NT*8 weight rows and a k range; its 8 warps cut that range in 8
// and the partial accumulators meet in shared memory, summed in warp order so
// results do not depend on scheduling.  What happens to the finished
// [m, NT*8] tile is the epilogue: fp32 split-k slice, bf16 store, SiLU*mul of
// paired gate/up rows, or the LM-head scan (temperature, noise, running
// max / sum-exp / argmax) that never writes a logit to memory.
#include "mdb_common.cuh"

namespace mdb {

enum SkinnyEpilogue { kEpiPartial = 0, kEpiBf16 = 1, kEpiSwiglu = 2, kEpiLmHead = 3 };

constexpr int kSkinnyWarps = 8;
constexpr int kSkinnyThreads = kSkinnyWarps * 32;

struct SkinnyArgs {
  const bf16* x;      // [m, k], row stride ldx
  const bf16* w;      // [n, k] row-major
  int64_t ldx;
  int m, n, k;
  int k_per_cta;      // multiple of 8*32
  // kEpiPartial
  float* partials;    // [gridDim.y][m][n]
  // kEpiBf16 / kEpiSwiglu
  bf16* y;
  int64_t ldy;
  int inter;          // kEpiSwiglu: n == 2*inter
  // kEpiLmHead
  const float* temperatures;  // [m / block]
  int block;
  int noise_mode;
  const float* noise;         // [m, n] when noise_mode == 1
  uint32_t seed, step;
  const uint32_t* step_dev;   // optional device-side addend to step
  float4* part_f;             // [n/32][m] (max, sumexp, best noisy, best logit)
  int* part_i;                // [n/32][m] best column
};

template <int MT, int NT, int EPI>
__global__ void __launch_bounds__(kSkinnyThreads)
gemm_skinny_kernel(const SkinnyArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int ROWS = MT * 16;  // activation rows (padded)
  constexpr int COLS = NT * 8;   // weight rows of this CTA
  // dynamic shared memory: red[8 warps][ROWS][COLS + 4] then tile[ROWS][COLS + 1]
  extern __shared__ __align__(16) float skinny_smem[];
  float (*red)[ROWS][COLS + 4] = reinterpret_cast<float (*)[ROWS][COLS + 4]>(skinny_smem);
  float (*tile)[COLS + 1] = reinterpret_cast<float (*)[COLS + 1]>(skinny_smem + kSkinnyWarps * ROWS * (COLS + 4));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int kw = a.k_per_cta / kSkinnyWarps;
  const int kbeg = blockIdx.y * a.k_per_cta + warp * kw;
  const int kend = min(kbeg + kw, a.k);

  // weight row of n-tile j for this lane
  const bf16* wrow[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    int row;
    if (EPI == kEpiSwiglu) {
      const int c0 = blockIdx.x * (COLS / 2);
      row = (j < NT / 2) ? c0 + 8 * j + g : a.inter + c0 + 8 * (j - NT / 2) + g;
    } else {
      row = blockIdx.x * COLS + 8 * j + g;
    }
    wrow[j] = a.w + static_cast<int64_t>(row) * a.k + 8 * t;
  }
  // activation rows g and g+8 of m-tile i (clamped: padded rows are never stored)
  const bf16* xrow[MT][2];
#pragma unroll
  for (int i = 0; i < MT; ++i) {
    xrow[i][0] = a.x + static_cast<int64_t>(min(16 * i + g, a.m - 1)) * a.ldx + 8 * t;
    xrow[i][1] = a.x + static_cast<int64_t>(min(16 * i + g + 8, a.m - 1)) * a.ldx + 8 * t;
  }

  float acc[MT][NT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

  constexpr int U = 2;  // 32-wide k steps fetched together
  for (int k0 = kbeg; k0 < kend; k0 += 32 * U) {
    uint4 wv[U][NT];
    uint4 xv[U][MT][2];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int kk = k0 + 32 * u;
      const bool live = kk < kend;
#pragma unroll
      for (int j = 0; j < NT; ++j) wv[u][j] = live ? ldg_stream16(wrow[j] + kk) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        xv[u][i][0] = live ? ldg_cached16(xrow[i][0] + kk) : make_uint4(0, 0, 0, 0);
        xv[u][i][1] = live ? ldg_cached16(xrow[i][1] + kk) : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          // lane's 8 contiguous k values: {0,1 | 2,3} -> first MMA, {4,5 | 6,7} -> second
          mma_bf16_16816(acc[i][j], xv[u][i][0].x, xv[u][i][1].x, xv[u][i][0].y, xv[u][i][1].y, wv[u][j].x,
                         wv[u][j].y);
          mma_bf16_16816(acc[i][j], xv[u][i][0].z, xv[u][i][1].z, xv[u][i][0].w, xv[u][i][1].w, wv[u][j].z,
                         wv[u][j].w);
        }
  }

  // meet in shared memory, sum in warp order
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      *reinterpret_cast<float2*>(&red[warp][16 * i + g][8 * j + 2 * t]) = make_float2(acc[i][j][0], acc[i][j][1]);
      *reinterpret_cast<float2*>(&red[warp][16 * i + g + 8][8 * j + 2 * t]) = make_float2(acc[i][j][2], acc[i][j][3]);
    }
  __syncthreads();
  for (int idx = threadIdx.x; idx < ROWS * COLS; idx += kSkinnyThreads) {
    const int r = idx / COLS, c = idx % COLS;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kSkinnyWarps; ++w) s += red[w][r][c];
    tile[r][c] = s;
  }
  __syncthreads();

  if (EPI == kEpiPartial) {
    const int n0 = blockIdx.x * COLS;
    for (int idx = threadIdx.x; idx < ROWS * COLS; idx += kSkinnyThreads) {
      const int r = idx / COLS, c = idx % COLS;
      if (r < a.m) a.partials[(static_cast<int64_t>(blockIdx.y) * a.m + r) * a.n + n0 + c] = tile[r][c];
    }
  } else if (EPI == kEpiBf16) {
    const int n0 = blockIdx.x * COLS;
    for (int idx = threadIdx.x; idx < ROWS * COLS / 2; idx += kSkinnyThreads) {
      const int r = idx / (COLS / 2), c = (idx % (COLS / 2)) * 2;
      if (r < a.m)
        *reinterpret_cast<uint32_t*>(a.y + r * a.ldy + n0 + c) = pack_bf16x2(tile[r][c], tile[r][c + 1]);
    }
  } else if (EPI == kEpiSwiglu) {
    constexpr int HALF = COLS / 2;
    const int c0 = blockIdx.x * HALF;
    for (int idx = threadIdx.x; idx < ROWS * HALF / 2; idx += kSkinnyThreads) {
      const int r = idx / (HALF / 2), c = (idx % (HALF / 2)) * 2;
      if (r < a.m) {
        float o[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float gt = bf16_round(tile[r][c + e]);        // gate_up_proj output is bf16
          const float up = bf16_round(tile[r][HALF + c + e]);
          const float s = gt * (1.0f / (1.0f + expf(-gt)));
          o[e] = bf16_round(s) * up;
        }
        *reinterpret_cast<uint32_t*>(a.y + r * a.ldy + c0 + c) = pack_bf16x2(o[0], o[1]);
      }
    }
  } else {  // kEpiLmHead: lane = vocabulary column of this CTA (COLS == 32)
    const int col = blockIdx.x * COLS + lane;
    const uint32_t step = a.step + (a.step_dev != nullptr ? *a.step_dev : 0u);
    for (int r = warp; r < a.m; r += kSkinnyWarps) {
      const float temp = a.temperatures[r / a.block];
      const float logit = bf16_round(tile[r][lane]) / temp;
      float noisy = logit;
      if (a.noise_mode == 1) noisy += a.noise[static_cast<int64_t>(r) * a.n + col];
      else if (a.noise_mode == 2) noisy += gumbel_noise(a.seed, step, r, col);
      const float mx = warp_max(logit);
      const float se = warp_sum(expf(logit - mx));
      // argmax of the noisy logit, lowest column wins a tie
      float bv = noisy, bl = logit;
      int bi = col;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const float ol = __shfl_xor_sync(0xffffffffu, bl, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bl = ol; bi = oi; }
      }
      if (lane == 0) {
        a.part_f[static_cast<int64_t>(blockIdx.x) * a.m + r] = make_float4(mx, se, bv, bl);
        a.part_i[static_cast<int64_t>(blockIdx.x) * a.m + r] = bi;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// sampler partial merge: one CTA per row over P partial records
// ---------------------------------------------------------------------------
struct SampleRec {
  float mx, se, bv, bl;
  int bi;
};

__device__ __forceinline__ void merge_rec(SampleRec& a, const SampleRec& b) {
  const float nm = fmaxf(a.mx, b.mx);
  const float sa = (a.mx == -INFINITY) ? 0.f : a.se * expf(a.mx - nm);
  const float sb = (b.mx == -INFINITY) ? 0.f : b.se * expf(b.mx - nm);
  a.se = sa + sb;
  a.mx = nm;
  if (b.bv > a.bv || (b.bv == a.bv && b.bi < a.bi)) { a.bv = b.bv; a.bl = b.bl; a.bi = b.bi; }
}

constexpr int kFinalizeThreads = 256;

__global__ void __launch_bounds__(kFinalizeThreads)
sampler_finalize_kernel(const float4* __restrict__ part_f, const int* __restrict__ part_i, int nparts, int m,
                        int32_t* __restrict__ x0_out, float* __restrict__ conf_out, const TpSignal tp) {
  pdl_launch_dependents();
  pdl_wait();
  tp_wait(tp);     // tensor-parallel pair: the peer's records of its vocabulary shard must have landed
  const int row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  SampleRec r = {-INFINITY, 0.f, -INFINITY, 0.f, 0x7fffffff};
  for (int p = threadIdx.x; p < nparts; p += kFinalizeThreads) {
    const float4 f = part_f[static_cast<int64_t>(p) * m + row];
    const SampleRec o = {f.x, f.y, f.z, f.w, part_i[static_cast<int64_t>(p) * m + row]};
    merge_rec(r, o);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    SampleRec t;
    t.mx = __shfl_xor_sync(0xffffffffu, r.mx, o);
    t.se = __shfl_xor_sync(0xffffffffu, r.se, o);
    t.bv = __shfl_xor_sync(0xffffffffu, r.bv, o);
    t.bl = __shfl_xor_sync(0xffffffffu, r.bl, o);
    t.bi = __shfl_xor_sync(0xffffffffu, r.bi, o);
    merge_rec(r, t);
  }
  __shared__ SampleRec sh[kFinalizeThreads / 32];
  if (lane == 0) sh[warp] = r;
  __syncthreads();
  if (threadIdx.x == 0) {
    SampleRec t = sh[0];
    for (int w = 1; w < kFinalizeThreads / 32; ++w) merge_rec(t, sh[w]);
    x0_out[row] = t.bi;
    conf_out[row] = expf(t.bl - t.mx) / t.se;
  }
}

// Scan of materialised bf16 logits: CTA = (column chunk of 1024, row).
constexpr int kScanCols = 1024;

__global__ void __launch_bounds__(256)
logits_scan_kernel(const bf16* __restrict__ logits, int64_t ld, int m, int vocab, const float* __restrict__ temperatures,
                   int block, int noise_mode, const float* __restrict__ noise, uint32_t seed, uint32_t step_base,
                   const uint32_t* __restrict__ step_dev, float4* __restrict__ part_f, int* __restrict__ part_i) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.y;
  const uint32_t step = step_base + (step_dev != nullptr ? *step_dev : 0u);
  const int c_begin = blockIdx.x * kScanCols;
  const float temp = temperatures[row / block];
  float mx = -INFINITY, se = 0.f, bv = -INFINITY, bl = 0.f;
  int bi = 0x7fffffff;
  for (int c = c_begin + threadIdx.x; c < min(c_begin + kScanCols, vocab); c += 256) {
    const float logit = __bfloat162float(logits[row * ld + c]) / temp;
    float noisy = logit;
    if (noise_mode == 1) noisy += noise[static_cast<int64_t>(row) * vocab + c];
    else if (noise_mode == 2) noisy += gumbel_noise(seed, step, row, c);
    const float nm = fmaxf(mx, logit);
    se = se * expf(mx - nm) + expf(logit - nm);
    mx = nm;
    if (noisy > bv || (noisy == bv && c < bi)) { bv = noisy; bl = logit; bi = c; }
  }
  __shared__ float4 sf[256];
  __shared__ int si[256];
  sf[threadIdx.x] = make_float4(mx, se, bv, bl);
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int stride = 128; stride > 0; stride >>= 1) {
    if (threadIdx.x < stride) {
      const float4 x = sf[threadIdx.x], y = sf[threadIdx.x + stride];
      const int xi = si[threadIdx.x], yi = si[threadIdx.x + stride];
      const float nm = fmaxf(x.x, y.x);
      const float sa = (x.x == -INFINITY) ? 0.f : x.y * expf(x.x - nm);
      const float sb = (y.x == -INFINITY) ? 0.f : y.y * expf(y.x - nm);
      float4 r = make_float4(nm, sa + sb, x.z, x.w);
      int ri = xi;
      if (y.z > x.z || (y.z == x.z && yi < xi)) { r.z = y.z; r.w = y.w; ri = yi; }
      sf[threadIdx.x] = r;
      si[threadIdx.x] = ri;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    part_f[static_cast<int64_t>(blockIdx.x) * m + row] = sf[0];
    part_i[static_cast<int64_t>(blockIdx.x) * m + row] = si[0];
  }
}

__global__ void gumbel_noise_kernel(float* __restrict__ out, int m, int vocab, uint32_t seed, uint32_t step) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = static_cast<int64_t>(m) * vocab;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x)
    out[idx] = gumbel_noise(seed, step, static_cast<uint32_t>(idx / vocab), static_cast<uint32_t>(idx % vocab));
}

// Unmask rule: one CTA per request, thread i = position i of the block.
__global__ void unmask_decide_kernel(int64_t* __restrict__ block_ids, const int32_t* __restrict__ x0,
                                     const float* __restrict__ conf, int block, int64_t mask_id, float threshold,
                                     int quota, uint8_t* __restrict__ transfer_out, int32_t* __restrict__ count_out) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sconf[128];
  const int req = blockIdx.x;
  const int i = threadIdx.x;
  const bool in_block = i < block;
  const int64_t id = in_block ? block_ids[static_cast<int64_t>(req) * block + i] : 0;
  const bool masked = in_block && id == mask_id;
  const float c = masked ? conf[static_cast<int64_t>(req) * block + i] : -INFINITY;
  sconf[i] = c;
  const int n_masked = __syncthreads_count(masked);
  if (n_masked == 0) {
    if (in_block) transfer_out[static_cast<int64_t>(req) * block + i] = 0;
    if (i == 0) count_out[req] = 0;
    return;
  }
  const bool hi = masked && c > threshold;
  const int n_hi = __syncthreads_count(hi);
  bool transfer;
  if (n_hi >= quota) {
    transfer = hi;
  } else {
    int rank = 0;
    for (int j = 0; j < block; ++j) {
      const float cj = sconf[j];
      rank += (cj > c || (cj == c && j < i)) ? 1 : 0;
    }
    transfer = masked && rank < quota;
  }
  const int n_transfer = __syncthreads_count(transfer);
  if (in_block) {
    transfer_out[static_cast<int64_t>(req) * block + i] = transfer ? 1 : 0;
    if (transfer) block_ids[static_cast<int64_t>(req) * block + i] = x0[static_cast<int64_t>(req) * block + i];
  }
  if (i == 0) count_out[req] = n_transfer;
}

}  // namespace mdb

using namespace mdb;

namespace {

// k range of one CTA: whole multiples of 8 warps * 32
int skinny_k_per_cta(int k, int ksplit) {
  const int unit = kSkinnyWarps * 32;
  int per = (k + ksplit - 1) / ksplit;
  return (per + unit - 1) / unit * unit;
}

template <int MT, int NT, int EPI>
int launch_skinny_inst(const SkinnyArgs& a, int ksplit, cudaStream_t st) {
  constexpr int ROWS = MT * 16, COLS = NT * 8;
  constexpr int smem = (kSkinnyWarps * ROWS * (COLS + 4) + ROWS * (COLS + 1)) * 4;
  static bool attr_set = false;  // one flag per instantiation
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_skinny_kernel<MT, NT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
        cudaSuccess)
      return MDB_ERR_CUDA;
    attr_set = true;
  }
  const int cols = (EPI == kEpiSwiglu) ? a.inter : a.n;
  const int per_cta = (EPI == kEpiSwiglu) ? COLS / 2 : COLS;
  dim3 grid(cols / per_cta, ksplit);
  return mdb_launch(gemm_skinny_kernel<MT, NT, EPI>, grid, dim3(kSkinnyThreads), smem, st, a);
}

template <int EPI>
int launch_skinny(SkinnyArgs& a, int ksplit, cudaStream_t st) {
  const int mt = (a.m + 15) / 16;
  a.k_per_cta = skinny_k_per_cta(a.k, ksplit);
  if (mt == 1) return launch_skinny_inst<1, 4, EPI>(a, ksplit, st);
  if (mt == 2) return launch_skinny_inst<2, 4, EPI>(a, ksplit, st);
  // 3 or 4 m-tiles: fewer weight rows per warp keeps the accumulators in
  // registers; the LM head keeps 32 columns per CTA (lane = column)
  return launch_skinny_inst<4, (EPI == kEpiLmHead) ? 4 : 2, EPI>(a, ksplit, st);
}

int check_skinny_common(const void* x, int64_t ldx, const void* w, int m, int n, int k) {
  MDB_REQUIRE(x && w, MDB_ERR_ARG);
  MDB_REQUIRE(m >= 1 && m <= 64, MDB_ERR_UNSUPPORTED);
  MDB_REQUIRE(n > 0 && k > 0 && ldx >= k, MDB_ERR_ARG);
  MDB_REQUIRE(n % 32 == 0 && k % 32 == 0, MDB_ERR_UNSUPPORTED);
  MDB_REQUIRE(ldx % 8 == 0 && mdb_aligned16(x) && mdb_aligned16(w), MDB_ERR_ALIGN);
  return MDB_OK;
}

}  // namespace

extern "C" {

int mdb_gumbel_noise(float* out, int m, int vocab, uint32_t seed, uint32_t step, mdb_stream_t stream) {
  MDB_REQUIRE(m >= 0 && vocab > 0, MDB_ERR_ARG);
  if (m == 0) return MDB_OK;
  MDB_REQUIRE(out != nullptr, MDB_ERR_ARG);
  const int64_t total = static_cast<int64_t>(m) * vocab;
  int blocks = static_cast<int>((total + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  return mdb_launch(gumbel_noise_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream), out, m, vocab,
                    seed, step);
}

int mdb_unmask_decide(int64_t* block_ids, const int32_t* x0, const float* conf, int bs, int block, int64_t mask_id,
                      float threshold, int quota, uint8_t* transfer_out, int32_t* count_out, mdb_stream_t stream) {
  MDB_REQUIRE(bs >= 0 && block > 0 && quota >= 1, MDB_ERR_ARG);
  if (bs == 0) return MDB_OK;
  MDB_REQUIRE(block_ids && x0 && conf && transfer_out && count_out, MDB_ERR_ARG);
  MDB_REQUIRE(block <= 128, MDB_ERR_UNSUPPORTED);
  const int threads = block <= 32 ? 32 : (block <= 64 ? 64 : 128);
  return mdb_launch(unmask_decide_kernel, dim3(bs), dim3(threads), 0, static_cast<cudaStream_t>(stream), block_ids, x0,
                    conf, block, mask_id, threshold, quota, transfer_out, count_out);
}

}  // extern "C"
