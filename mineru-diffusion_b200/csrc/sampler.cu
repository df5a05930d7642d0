// Sampler kernels behind the LM head: merge of the per-tile (max, sum-exp,
// best noisy value, its logit, its index) records the LM-head epilogues write,
// the scan of materialised bf16 logits, the counter-based Gumbel noise dump and
// the unmask rule of the block-diffusion sampler.  All latency-bound: a few MB
// at most.
#include "mdb_common.cuh"

namespace mdb {

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
                                     int quota_all, const int32_t* __restrict__ quotas,
                                     uint8_t* __restrict__ transfer_out, int32_t* __restrict__ count_out,
                                     uint32_t* __restrict__ status_out) {
  pdl_launch_dependents();
  pdl_wait();
  // last kernel of a step: hand the status word the step's kernels may have raised to the host's result copy
  if (status_out != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *status_out = atomicExch(&g_device_status, 0u);
  __shared__ float sconf[128];
  const int req = blockIdx.x;
  const int i = threadIdx.x;
  const int quota = quotas != nullptr ? max(0, quotas[req]) : quota_all;   // per request where the schedule differs
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
                      float threshold, int quota, const int32_t* quotas, uint8_t* transfer_out, int32_t* count_out,
                      uint32_t* status_out, mdb_stream_t stream) {
  MDB_REQUIRE(bs >= 0 && block > 0 && quota >= 0, MDB_ERR_ARG);
  if (bs == 0) return MDB_OK;
  MDB_REQUIRE(block_ids && x0 && conf && transfer_out && count_out, MDB_ERR_ARG);
  MDB_REQUIRE(block <= 128, MDB_ERR_UNSUPPORTED);
  const int threads = block <= 32 ? 32 : (block <= 64 ? 64 : 128);
  return mdb_launch(unmask_decide_kernel, dim3(bs), dim3(threads), 0, static_cast<cudaStream_t>(stream), block_ids, x0,
                    conf, block, mask_id, threshold, quota, quotas, transfer_out, count_out, status_out);
}

}  // extern "C"
