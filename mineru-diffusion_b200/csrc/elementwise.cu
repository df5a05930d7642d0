// Memory-bound row kernels of the decode step: paged KV commit, RMSNorm with
// residual add, per-head q/k norm + rotary + KV store, SiLU*mul, row gather.
// All are HBM/L2-bound copies with a little fp32 math; 16-byte accesses, one
// row (or one head) per warp/CTA, no shared-memory staging needed.
#include "mdb_common.cuh"

namespace mdb {

// ---------------------------------------------------------------------------
// KV commit: one CTA per token row, K and V rows copied in 16-byte chunks.
// ---------------------------------------------------------------------------
__global__ void kv_commit_kernel(const bf16* __restrict__ key, int64_t key_stride, const bf16* __restrict__ value,
                                 int64_t value_stride, bf16* __restrict__ k_cache, bf16* __restrict__ v_cache,
                                 const int32_t* __restrict__ slot_mapping, int row_elems, int64_t num_slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x;
  const int slot = slot_mapping[i];
  if (slot == -1) return;
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) report_status(MDB_STATUS_BAD_SLOT);
    return;
  }
  const int chunks = row_elems >> 3;
  const uint4* ks = reinterpret_cast<const uint4*>(key + static_cast<int64_t>(i) * key_stride);
  const uint4* vs = reinterpret_cast<const uint4*>(value + static_cast<int64_t>(i) * value_stride);
  uint4* kd = reinterpret_cast<uint4*>(k_cache + static_cast<int64_t>(slot) * row_elems);
  uint4* vd = reinterpret_cast<uint4*>(v_cache + static_cast<int64_t>(slot) * row_elems);
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    kd[c] = ks[c];
    vd[c] = vs[c];
  }
}

// ---------------------------------------------------------------------------
// RMSNorm (+ residual add, + split-K reduction of the producing GEMM)
// ---------------------------------------------------------------------------
constexpr int kNormThreads = 256;
constexpr int kNormMaxChunks = 4;  // h <= 256 * 4 * 8 = 8192

// PARTIALS: the input row is the sum of fp32 slices (short steps; latency-bound, loads batched) or a bf16 row.
template <bool PARTIALS>
__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ x2, const float* __restrict__ partials, int nparts,
                   const bf16* __restrict__ residual_in, const bf16* __restrict__ weight, float eps,
                   bf16* __restrict__ y_out, bf16* __restrict__ residual_out, int m, int h, const TpSignal tp) {
  if (threadIdx.x == 0) trace_event(10, 0);
  pdl_launch_dependents();
  pdl_wait();
  tp_wait(tp);     // tensor-parallel pair: the peer's slices must have landed
  if (threadIdx.x == 0) trace_event(10, 1);
  const int row = blockIdx.x;
  const int chunks = h >> 3;
  const int64_t row_off = static_cast<int64_t>(row) * h;
  float v[kNormMaxChunks][8];
  float sumsq = 0.f;
#pragma unroll
  for (int it = 0; it < kNormMaxChunks; ++it) {
    const int c = threadIdx.x + it * kNormThreads;
    if (c < chunks) {
      float a[8];
      if (PARTIALS) {
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = 0.f;
        // slices are summed in slice order; the loads of eight slices go out together (one L2 round trip
        // instead of eight dependent ones: this kernel is pure latency at 32 rows)
        const int64_t pstride = static_cast<int64_t>(m) * h;
        const float* src0 = partials + static_cast<int64_t>(row) * h + c * 8;
        for (int p0 = 0; p0 < nparts; p0 += 8) {
          float4 lo[8], hi[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (p0 + i < nparts) {
              const float4* src = reinterpret_cast<const float4*>(src0 + (p0 + i) * pstride);
              lo[i] = src[0];
              hi[i] = src[1];
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (p0 + i < nparts) {
              a[0] += lo[i].x; a[1] += lo[i].y; a[2] += lo[i].z; a[3] += lo[i].w;
              a[4] += hi[i].x; a[5] += hi[i].y; a[6] += hi[i].z; a[7] += hi[i].w;
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = bf16_round(a[j]);  // the rounding F.linear applies to its output
      } else {
        const uint4 u = *reinterpret_cast<const uint4*>(x + row_off + c * 8);
        float2 f;
        f = unpack_bf16x2(u.x); a[0] = f.x; a[1] = f.y;
        f = unpack_bf16x2(u.y); a[2] = f.x; a[3] = f.y;
        f = unpack_bf16x2(u.z); a[4] = f.x; a[5] = f.y;
        f = unpack_bf16x2(u.w); a[6] = f.x; a[7] = f.y;
        if (x2 != nullptr) {
          // tensor-parallel pair: the other rank's partial output; the sum is rounded to bf16 as the
          // all-reduce of two bf16 tensors rounds it (a + b is the same on both ranks)
          const uint4 w2 = *reinterpret_cast<const uint4*>(x2 + row_off + c * 8);
          f = unpack_bf16x2(w2.x); a[0] = bf16_round(a[0] + f.x); a[1] = bf16_round(a[1] + f.y);
          f = unpack_bf16x2(w2.y); a[2] = bf16_round(a[2] + f.x); a[3] = bf16_round(a[3] + f.y);
          f = unpack_bf16x2(w2.z); a[4] = bf16_round(a[4] + f.x); a[5] = bf16_round(a[5] + f.y);
          f = unpack_bf16x2(w2.w); a[6] = bf16_round(a[6] + f.x); a[7] = bf16_round(a[7] + f.y);
        }
      }
      if (residual_in != nullptr) {
        const uint4 u = *reinterpret_cast<const uint4*>(residual_in + row_off + c * 8);
        float2 f;
        f = unpack_bf16x2(u.x); a[0] += f.x; a[1] += f.y;
        f = unpack_bf16x2(u.y); a[2] += f.x; a[3] += f.y;
        f = unpack_bf16x2(u.z); a[4] += f.x; a[5] += f.y;
        f = unpack_bf16x2(u.w); a[6] += f.x; a[7] += f.y;
      }
      if (residual_out != nullptr) {
        uint4 o;
        o.x = pack_bf16x2(a[0], a[1]); o.y = pack_bf16x2(a[2], a[3]);
        o.z = pack_bf16x2(a[4], a[5]); o.w = pack_bf16x2(a[6], a[7]);
        *reinterpret_cast<uint4*>(residual_out + row_off + c * 8) = o;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[it][j] = a[j];
        sumsq += a[j] * a[j];
      }
    }
  }
  __shared__ float red[kNormThreads / 32];
  sumsq = warp_sum(sumsq);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sumsq;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < kNormThreads / 32; ++w) total += red[w];
  const float rstd = 1.0f / sqrtf(total / static_cast<float>(h) + eps);
#pragma unroll
  for (int it = 0; it < kNormMaxChunks; ++it) {
    const int c = threadIdx.x + it * kNormThreads;
    if (c < chunks) {
      const uint4 wu = *reinterpret_cast<const uint4*>(weight + c * 8);
      float w[8];
      float2 f;
      f = unpack_bf16x2(wu.x); w[0] = f.x; w[1] = f.y;
      f = unpack_bf16x2(wu.y); w[2] = f.x; w[3] = f.y;
      f = unpack_bf16x2(wu.z); w[4] = f.x; w[5] = f.y;
      f = unpack_bf16x2(wu.w); w[6] = f.x; w[7] = f.y;
      float r[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) r[j] = bf16_round(v[it][j] * rstd) * w[j];  // bf16 * bf16, rounded below
      uint4 o;
      o.x = pack_bf16x2(r[0], r[1]); o.y = pack_bf16x2(r[2], r[3]);
      o.z = pack_bf16x2(r[4], r[5]); o.w = pack_bf16x2(r[6], r[7]);
      *reinterpret_cast<uint4*>(y_out + row_off + c * 8) = o;
    }
  }
  if (threadIdx.x == 0) trace_event(10, 2);
}

// Many-row steps (prefill, batched decode): one warp per row and no block-wide barrier.  Lane l owns the 16-byte
// chunks l, l + 32, ... of its row, so a warp reads contiguous 512-byte segments and keeps NCH loads per input in
// flight per lane; the arithmetic per element is that of add_rmsnorm_kernel, only the order of the fp32 sum of
// squares differs (per lane, then across the warp).
constexpr int kNormRowsWarps = 8;

__device__ __forceinline__ void unpack8(const uint4& u, float* a) {
  float2 f;
  f = unpack_bf16x2(u.x); a[0] = f.x; a[1] = f.y;
  f = unpack_bf16x2(u.y); a[2] = f.x; a[3] = f.y;
  f = unpack_bf16x2(u.z); a[4] = f.x; a[5] = f.y;
  f = unpack_bf16x2(u.w); a[6] = f.x; a[7] = f.y;
}

template <int NCH>
__global__ void __launch_bounds__(kNormRowsWarps * 32)
add_rmsnorm_rows_kernel(const bf16* __restrict__ x, const bf16* __restrict__ x2, const bf16* __restrict__ residual_in,
                        const bf16* __restrict__ weight, float eps, bf16* __restrict__ y_out,
                        bf16* __restrict__ residual_out, int m, const TpSignal tp) {
  pdl_launch_dependents();
  pdl_wait();
  tp_wait(tp);     // tensor-parallel pair: the peer's rows must have landed
  constexpr int h = NCH * 256;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kNormRowsWarps + (threadIdx.x >> 5);
  if (row >= m) return;
  const int64_t row_off = static_cast<int64_t>(row) * h;
  uint4 ux[NCH], ur[NCH];
#pragma unroll
  for (int i = 0; i < NCH; ++i) ux[i] = *reinterpret_cast<const uint4*>(x + row_off + (lane + 32 * i) * 8);
  if (residual_in != nullptr) {
#pragma unroll
    for (int i = 0; i < NCH; ++i) ur[i] = *reinterpret_cast<const uint4*>(residual_in + row_off + (lane + 32 * i) * 8);
  }
  float v[NCH][8];
  float sumsq = 0.f;
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    float a[8];
    unpack8(ux[i], a);
    if (x2 != nullptr) {
      // tensor-parallel pair: bf16(own + peer), what the all-reduce of two bf16 tensors yields on both ranks
      float b[8];
      unpack8(*reinterpret_cast<const uint4*>(x2 + row_off + (lane + 32 * i) * 8), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = bf16_round(a[j] + b[j]);
    }
    if (residual_in != nullptr) {
      float r[8];
      unpack8(ur[i], r);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += r[j];
    }
    if (residual_out != nullptr) {
      uint4 o;
      o.x = pack_bf16x2(a[0], a[1]); o.y = pack_bf16x2(a[2], a[3]);
      o.z = pack_bf16x2(a[4], a[5]); o.w = pack_bf16x2(a[6], a[7]);
      *reinterpret_cast<uint4*>(residual_out + row_off + (lane + 32 * i) * 8) = o;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[i][j] = a[j];
      sumsq += a[j] * a[j];
    }
  }
  sumsq = warp_sum(sumsq);
  const float rstd = 1.0f / sqrtf(sumsq / static_cast<float>(h) + eps);
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    float w[8];
    unpack8(*reinterpret_cast<const uint4*>(weight + (lane + 32 * i) * 8), w);
    float r[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = bf16_round(v[i][j] * rstd) * w[j];  // bf16 * bf16, rounded below
    uint4 o;
    o.x = pack_bf16x2(r[0], r[1]); o.y = pack_bf16x2(r[2], r[3]);
    o.z = pack_bf16x2(r[4], r[5]); o.w = pack_bf16x2(r[6], r[7]);
    *reinterpret_cast<uint4*>(y_out + row_off + (lane + 32 * i) * 8) = o;
  }
}

template <int NCH>
static int launch_add_rmsnorm_rows(const void* x, const void* x2, const void* residual_in, const void* weight, float eps,
                                   void* y_out, void* residual_out, int m, const TpSignal& tp, mdb_stream_t stream) {
  return mdb_launch(add_rmsnorm_rows_kernel<NCH>, dim3((m + kNormRowsWarps - 1) / kNormRowsWarps),
                    dim3(kNormRowsWarps * 32), 0, static_cast<cudaStream_t>(stream), static_cast<const bf16*>(x),
                    static_cast<const bf16*>(x2), static_cast<const bf16*>(residual_in),
                    static_cast<const bf16*>(weight), eps, static_cast<bf16*>(y_out), static_cast<bf16*>(residual_out),
                    m, tp);
}

// ---------------------------------------------------------------------------
// q/k per-head RMSNorm + rotary + KV store; one warp per (token, head).
// Lane l owns head elements {2l, 2l+1, 2l+64, 2l+65}: the two halves the
// NeoX rotation pairs up.
// ---------------------------------------------------------------------------
constexpr int kRopeWarps = 4;

// One (token, head) of the fused qkv output: per-head RMSNorm for q and k heads, rotary embedding, store of q into
// q_out and of k / v into the contiguous outputs and/or the paged cache.  Executed by one warp.
__device__ __forceinline__ void qknorm_rope_commit_warp(
    int token, int head, int lane, const bf16* __restrict__ qkv, int64_t ld_qkv, const float* __restrict__ partials,
    int nparts, const int64_t* __restrict__ positions, const float* __restrict__ rope_table, int max_pos,
    const bf16* __restrict__ q_norm_w, const bf16* __restrict__ k_norm_w, float eps,
    const int32_t* __restrict__ slot_mapping, bf16* __restrict__ q_out, bf16* __restrict__ k_out,
    bf16* __restrict__ v_out, bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, int64_t num_slots, int m, int hq,
    int hkv) {
  const int nheads = hq + 2 * hkv;
  if (head >= nheads) return;
  const int ncols = nheads * kHeadDim;
  const int col0 = head * kHeadDim + 2 * lane;

  float a[4];  // elements 2l, 2l+1, 2l+64, 2l+65
  if (partials != nullptr) {
    a[0] = a[1] = a[2] = a[3] = 0.f;
    const int64_t pstride = static_cast<int64_t>(m) * ncols;
    const float* src0 = partials + static_cast<int64_t>(token) * ncols + col0;
    for (int p0 = 0; p0 < nparts; p0 += 8) {      // eight slices' loads in flight together, summed in slice order
      float2 lo[8], hi[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (p0 + i < nparts) {
          lo[i] = *reinterpret_cast<const float2*>(src0 + (p0 + i) * pstride);
          hi[i] = *reinterpret_cast<const float2*>(src0 + (p0 + i) * pstride + 64);
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (p0 + i < nparts) { a[0] += lo[i].x; a[1] += lo[i].y; a[2] += hi[i].x; a[3] += hi[i].y; }
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) a[j] = bf16_round(a[j]);
  } else {
    const bf16* src = qkv + static_cast<int64_t>(token) * ld_qkv + col0;
    const float2 lo = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(src));
    const float2 hi = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(src + 64));
    a[0] = lo.x; a[1] = lo.y; a[2] = hi.x; a[3] = hi.y;
  }

  const bool is_q = head < hq;
  const bool is_k = !is_q && head < hq + hkv;
  if (is_q || is_k) {
    float ss = a[0] * a[0] + a[1] * a[1] + a[2] * a[2] + a[3] * a[3];
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / static_cast<float>(kHeadDim) + eps);
    const bf16* nw = is_q ? q_norm_w : k_norm_w;
    const float2 wlo = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(nw + 2 * lane));
    const float2 whi = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(nw + 2 * lane + 64));
    a[0] = bf16_round(bf16_round(a[0] * rstd) * wlo.x);
    a[1] = bf16_round(bf16_round(a[1] * rstd) * wlo.y);
    a[2] = bf16_round(bf16_round(a[2] * rstd) * whi.x);
    a[3] = bf16_round(bf16_round(a[3] * rstd) * whi.y);
    const int64_t pos = positions[token];
    if (pos >= 0 && pos < max_pos) {
      const float* cs = rope_table + pos * kHeadDim;
      const float2 c = *reinterpret_cast<const float2*>(cs + 2 * lane);
      const float2 s = *reinterpret_cast<const float2*>(cs + 64 + 2 * lane);
      // products rounded separately, as un-fused fp32 tensor ops do
      const float y0 = __fsub_rn(__fmul_rn(a[0], c.x), __fmul_rn(a[2], s.x));
      const float y2 = __fadd_rn(__fmul_rn(a[2], c.x), __fmul_rn(a[0], s.x));
      const float y1 = __fsub_rn(__fmul_rn(a[1], c.y), __fmul_rn(a[3], s.y));
      const float y3 = __fadd_rn(__fmul_rn(a[3], c.y), __fmul_rn(a[1], s.y));
      a[0] = y0; a[1] = y1; a[2] = y2; a[3] = y3;
    } else if (lane == 0) {
      report_status(MDB_STATUS_BAD_POSITION);
    }
  }
  const uint32_t lo = pack_bf16x2(a[0], a[1]);
  const uint32_t hi = pack_bf16x2(a[2], a[3]);

  if (is_q) {
    bf16* dst = q_out + (static_cast<int64_t>(token) * hq + head) * kHeadDim + 2 * lane;
    *reinterpret_cast<uint32_t*>(dst) = lo;
    *reinterpret_cast<uint32_t*>(dst + 64) = hi;
    return;
  }
  const int kvh = is_k ? head - hq : head - hq - hkv;
  bf16* contiguous = is_k ? k_out : v_out;
  if (contiguous != nullptr) {
    bf16* dst = contiguous + (static_cast<int64_t>(token) * hkv + kvh) * kHeadDim + 2 * lane;
    *reinterpret_cast<uint32_t*>(dst) = lo;
    *reinterpret_cast<uint32_t*>(dst + 64) = hi;
  }
  if (slot_mapping != nullptr) {
    const int slot = slot_mapping[token];
    if (slot == -1) return;
    if (slot < 0 || slot >= num_slots) {
      if (lane == 0) report_status(MDB_STATUS_BAD_SLOT);
      return;
    }
    bf16* cache = is_k ? k_cache : v_cache;
    bf16* dst = cache + (static_cast<int64_t>(slot) * hkv + kvh) * kHeadDim + 2 * lane;
    *reinterpret_cast<uint32_t*>(dst) = lo;
    *reinterpret_cast<uint32_t*>(dst + 64) = hi;
  }
}

__global__ void __launch_bounds__(kRopeWarps * 32)
qknorm_rope_commit_kernel(const bf16* __restrict__ qkv, int64_t ld_qkv, const float* __restrict__ partials, int nparts,
                          const int64_t* __restrict__ positions, const float* __restrict__ rope_table, int max_pos,
                          const bf16* __restrict__ q_norm_w, const bf16* __restrict__ k_norm_w, float eps,
                          const int32_t* __restrict__ slot_mapping, bf16* __restrict__ q_out,
                          bf16* __restrict__ k_out, bf16* __restrict__ v_out, bf16* __restrict__ k_cache,
                          bf16* __restrict__ v_cache, int64_t num_slots, int m, int hq, int hkv) {
  if (threadIdx.x == 0) trace_event(32, 0);
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) trace_event(32, 1);
  qknorm_rope_commit_warp(blockIdx.x, blockIdx.y * kRopeWarps + (threadIdx.x >> 5), threadIdx.x & 31, qkv, ld_qkv,
                          partials, nparts, positions, rope_table, max_pos, q_norm_w, k_norm_w, eps, slot_mapping,
                          q_out, k_out, v_out, k_cache, v_cache, num_slots, m, hq, hkv);
  if (threadIdx.x == 0) trace_event(32, 2);
}

// ---------------------------------------------------------------------------
// SiLU*mul on a materialised gate|up matrix
// ---------------------------------------------------------------------------
__device__ __forceinline__ float silu_mul_bf16(float g, float u) {
  const float s = g * (1.0f / (1.0f + expf(-g)));
  return bf16_round(s) * u;  // bf16 * bf16; caller rounds
}

__global__ void silu_mul_kernel(const bf16* __restrict__ gate_up, int64_t ld_in, bf16* __restrict__ act,
                                int64_t ld_act, int m, int inter) {
  pdl_launch_dependents();
  pdl_wait();
  const int chunks = inter >> 3;
  const int64_t total = static_cast<int64_t>(m) * chunks;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(idx / chunks);
    const int c = static_cast<int>(idx % chunks);
    const bf16* src = gate_up + row * ld_in + c * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(src);
    const uint4 u = *reinterpret_cast<const uint4*>(src + inter);
    const uint32_t gs[4] = {g.x, g.y, g.z, g.w};
    const uint32_t us[4] = {u.x, u.y, u.z, u.w};
    uint32_t os[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 gf = unpack_bf16x2(gs[j]);
      const float2 uf = unpack_bf16x2(us[j]);
      os[j] = pack_bf16x2(silu_mul_bf16(gf.x, uf.x), silu_mul_bf16(gf.y, uf.y));
    }
    *reinterpret_cast<uint4*>(act + row * ld_act + c * 8) = make_uint4(os[0], os[1], os[2], os[3]);
  }
}

// ---------------------------------------------------------------------------
// Row gather (token embedding, last-block row pick)
// ---------------------------------------------------------------------------
__global__ void gather_rows_kernel(const bf16* __restrict__ table, int64_t num_rows, const int64_t* __restrict__ ids,
                                   bf16* __restrict__ out, int h) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x;
  const int64_t id = ids[i];
  const int chunks = h >> 3;
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<int64_t>(i) * h);
  if (id < 0 || id >= num_rows) {
    if (threadIdx.x == 0) report_status(MDB_STATUS_BAD_TOKEN);
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) dst[c] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(table + id * h);
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) dst[c] = src[c];
}

}  // namespace mdb

using namespace mdb;

extern "C" {

const char* mdb_strerror(int code) {
  switch (code) {
    case MDB_OK: return "ok";
    case MDB_ERR_ARG: return "invalid argument (null pointer, non-positive size or inconsistent dimensions)";
    case MDB_ERR_ALIGN: return "pointer or stride is not 16-byte aligned";
    case MDB_ERR_UNSUPPORTED: return "shape not supported by the sm_100a kernels";
    case MDB_ERR_CUDA: return "CUDA runtime refused the launch";
    case MDB_ERR_WORKSPACE: return "workspace too small";
    case MDB_ERR_STATIC_LIMIT:
      return "request exceeds the fixed scratch array of the allocation-free entry point (lower nsplit or the batch)";
    default: return "unknown error code";
  }
}

int mdb_version(void) { return 101; }

int mdb_set_trace(void* buffer, int64_t bytes) {
  TraceBuf t;
  t.data = static_cast<unsigned long long*>(buffer);
  t.capacity = buffer != nullptr && bytes >= 32 ? static_cast<unsigned int>((bytes - 8) / 24) : 0;
  if (t.capacity == 0) t.data = nullptr;
  return cudaMemcpyToSymbol(g_trace, &t, sizeof(t)) == cudaSuccess ? MDB_OK : MDB_ERR_CUDA;
}

int mdb_set_option(int option, int value) {
  switch (option) {
    case MDB_OPT_PDL: g_opt_pdl = value ? 1 : 0; return MDB_OK;
    case MDB_OPT_GEMM_PAIR:
      if (value < 0 || value > 2) return MDB_ERR_ARG;
      g_opt_gemm_pair = value;
      return MDB_OK;
    case MDB_OPT_WAIT_LIMIT_US: {
      if (value < 1) return MDB_ERR_ARG;
      const unsigned long long ns = static_cast<unsigned long long>(value) * 1000ull;
      if (cudaMemcpyToSymbol(g_wait_limit_ns, &ns, sizeof(ns)) != cudaSuccess) return MDB_ERR_CUDA;   // current device
      g_opt_wait_limit_us = value;
      return MDB_OK;
    }
    default: return MDB_ERR_ARG;
  }
}

int mdb_get_option(int option) {
  switch (option) {
    case MDB_OPT_PDL: return g_opt_pdl;
    case MDB_OPT_GEMM_PAIR: return g_opt_gemm_pair;
    case MDB_OPT_WAIT_LIMIT_US: return g_opt_wait_limit_us;
    default: return MDB_ERR_ARG;
  }
}

int mdb_last_device_status(unsigned int* out, int clear) {
  MDB_REQUIRE(out != nullptr, MDB_ERR_ARG);
  if (cudaDeviceSynchronize() != cudaSuccess) return MDB_ERR_CUDA;
  if (cudaMemcpyFromSymbol(out, g_device_status, sizeof(unsigned int)) != cudaSuccess) return MDB_ERR_CUDA;
  if (clear) {
    const unsigned int zero = 0;
    if (cudaMemcpyToSymbol(g_device_status, &zero, sizeof(unsigned int)) != cudaSuccess) return MDB_ERR_CUDA;
  }
  return MDB_OK;
}

int mdb_kv_commit(const void* key, int64_t key_stride, const void* value, int64_t value_stride, void* k_cache,
                  void* v_cache, const int32_t* slot_mapping, int n_tokens, int row_elems, int64_t num_slots,
                  mdb_stream_t stream) {
  MDB_REQUIRE(n_tokens >= 0 && row_elems > 0 && num_slots > 0, MDB_ERR_ARG);
  if (n_tokens == 0) return MDB_OK;
  MDB_REQUIRE(key && value && k_cache && v_cache && slot_mapping, MDB_ERR_ARG);
  MDB_REQUIRE(row_elems % 8 == 0, MDB_ERR_UNSUPPORTED);
  MDB_REQUIRE(key_stride >= row_elems && value_stride >= row_elems, MDB_ERR_ARG);
  MDB_REQUIRE(key_stride % 8 == 0 && value_stride % 8 == 0, MDB_ERR_ALIGN);
  MDB_REQUIRE(mdb_aligned16(key) && mdb_aligned16(value) && mdb_aligned16(k_cache) && mdb_aligned16(v_cache),
              MDB_ERR_ALIGN);
  const int threads = row_elems / 8 >= 128 ? 128 : 64;
  return mdb_launch(kv_commit_kernel, dim3(n_tokens), dim3(threads), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const bf16*>(key), key_stride, static_cast<const bf16*>(value), value_stride,
                    static_cast<bf16*>(k_cache), static_cast<bf16*>(v_cache), slot_mapping, row_elems, num_slots);
}

static int add_rmsnorm_impl(const void* x, const void* x2, const float* partials, int nparts, const void* residual_in,
                            const void* weight, float eps, void* y_out, void* residual_out, int m, int h,
                            const TpSignal& tp, mdb_stream_t stream) {
  MDB_REQUIRE(m >= 0 && h > 0, MDB_ERR_ARG);
  if (m == 0) return MDB_OK;
  MDB_REQUIRE((x != nullptr) != (partials != nullptr), MDB_ERR_ARG);
  MDB_REQUIRE(partials == nullptr || nparts >= 1, MDB_ERR_ARG);
  MDB_REQUIRE(weight && y_out, MDB_ERR_ARG);
  MDB_REQUIRE(h % 8 == 0 && h <= kNormThreads * kNormMaxChunks * 8, MDB_ERR_UNSUPPORTED);
  MDB_REQUIRE(mdb_aligned16(x) && mdb_aligned16(partials) && mdb_aligned16(residual_in) && mdb_aligned16(weight) &&
                  mdb_aligned16(y_out) && mdb_aligned16(residual_out),
              MDB_ERR_ALIGN);
  if (partials == nullptr && m > 64) {
    // many rows: a warp per row (row widths that are a power-of-two multiple of 256 up to 2048)
    switch (h) {
      case 256: return launch_add_rmsnorm_rows<1>(x, x2, residual_in, weight, eps, y_out, residual_out, m, tp, stream);
      case 512: return launch_add_rmsnorm_rows<2>(x, x2, residual_in, weight, eps, y_out, residual_out, m, tp, stream);
      case 1024: return launch_add_rmsnorm_rows<4>(x, x2, residual_in, weight, eps, y_out, residual_out, m, tp, stream);
      case 2048: return launch_add_rmsnorm_rows<8>(x, x2, residual_in, weight, eps, y_out, residual_out, m, tp, stream);
      default: break;
    }
  }
  if (partials != nullptr)
    return mdb_launch(add_rmsnorm_kernel<true>, dim3(m), dim3(kNormThreads), 0, static_cast<cudaStream_t>(stream),
                      static_cast<const bf16*>(x), static_cast<const bf16*>(x2), partials, nparts,
                      static_cast<const bf16*>(residual_in), static_cast<const bf16*>(weight), eps,
                      static_cast<bf16*>(y_out), static_cast<bf16*>(residual_out), m, h, tp);
  return mdb_launch(add_rmsnorm_kernel<false>, dim3(m), dim3(kNormThreads), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const bf16*>(x), static_cast<const bf16*>(x2), partials, nparts,
                    static_cast<const bf16*>(residual_in), static_cast<const bf16*>(weight), eps,
                    static_cast<bf16*>(y_out), static_cast<bf16*>(residual_out), m, h, tp);
}

int mdb_add_rmsnorm(const void* x, const float* partials, int nparts, const void* residual_in, const void* weight,
                    float eps, void* y_out, void* residual_out, int m, int h, mdb_stream_t stream) {
  const TpSignal none = {nullptr, nullptr, 0, 0, nullptr};
  return add_rmsnorm_impl(x, nullptr, partials, nparts, residual_in, weight, eps, y_out, residual_out, m, h, none, stream);
}

int mdb_add_rmsnorm_tp(const void* x, const float* partials, int nparts, const void* residual_in, const void* weight,
                       float eps, void* y_out, void* residual_out, int m, int h, const uint32_t* wait_flags,
                       int wait_count, uint32_t tag, const uint32_t* epoch, mdb_stream_t stream) {
  MDB_REQUIRE(wait_flags && epoch && wait_count > 0 && tag >= 1 && tag <= 255, MDB_ERR_ARG);
  const TpSignal tp = {nullptr, wait_flags, wait_count, tag, epoch};
  return add_rmsnorm_impl(x, nullptr, partials, nparts, residual_in, weight, eps, y_out, residual_out, m, h, tp, stream);
}

int mdb_add_rmsnorm_tp_rows(const void* x, const void* x_peer, const void* residual_in, const void* weight, float eps,
                            void* y_out, void* residual_out, int m, int h, const uint32_t* wait_flags, int wait_count,
                            uint32_t tag, const uint32_t* epoch, mdb_stream_t stream) {
  MDB_REQUIRE(x && x_peer && wait_flags && epoch && wait_count > 0 && tag >= 1 && tag <= 255, MDB_ERR_ARG);
  MDB_REQUIRE(mdb_aligned16(x_peer), MDB_ERR_ALIGN);
  const TpSignal tp = {nullptr, wait_flags, wait_count, tag, epoch};
  return add_rmsnorm_impl(x, x_peer, nullptr, 0, residual_in, weight, eps, y_out, residual_out, m, h, tp, stream);
}

int mdb_qknorm_rope_commit(const void* qkv, int64_t ld_qkv, const float* partials, int nparts,
                           const int64_t* positions, const float* rope_table, int max_pos, const void* q_norm_w,
                           const void* k_norm_w, float eps, const int32_t* slot_mapping, void* q_out, void* k_out,
                           void* v_out, void* k_cache, void* v_cache, int64_t num_slots, int m, int hq, int hkv,
                           mdb_stream_t stream) {
  MDB_REQUIRE(m >= 0 && hq > 0 && hkv > 0 && max_pos > 0, MDB_ERR_ARG);
  if (m == 0) return MDB_OK;
  MDB_REQUIRE((qkv != nullptr) != (partials != nullptr), MDB_ERR_ARG);
  MDB_REQUIRE(partials == nullptr || nparts >= 1, MDB_ERR_ARG);
  MDB_REQUIRE(positions && rope_table && q_norm_w && k_norm_w && q_out, MDB_ERR_ARG);
  MDB_REQUIRE(slot_mapping == nullptr || (k_cache && v_cache && num_slots > 0), MDB_ERR_ARG);
  MDB_REQUIRE(qkv == nullptr || (ld_qkv >= static_cast<int64_t>(hq + 2 * hkv) * kHeadDim && ld_qkv % 2 == 0),
              MDB_ERR_ARG);
  MDB_REQUIRE(mdb_aligned16(qkv) && mdb_aligned16(partials) && mdb_aligned16(rope_table) && mdb_aligned16(q_out) &&
                  mdb_aligned16(k_out) && mdb_aligned16(v_out) && mdb_aligned16(k_cache) && mdb_aligned16(v_cache) &&
                  mdb_aligned16(q_norm_w) && mdb_aligned16(k_norm_w),
              MDB_ERR_ALIGN);
  const int nheads = hq + 2 * hkv;
  dim3 grid(m, (nheads + kRopeWarps - 1) / kRopeWarps);
  return mdb_launch(qknorm_rope_commit_kernel, grid, dim3(kRopeWarps * 32), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const bf16*>(qkv), ld_qkv, partials, nparts, positions, rope_table, max_pos,
                    static_cast<const bf16*>(q_norm_w), static_cast<const bf16*>(k_norm_w), eps, slot_mapping,
                    static_cast<bf16*>(q_out), static_cast<bf16*>(k_out), static_cast<bf16*>(v_out),
                    static_cast<bf16*>(k_cache), static_cast<bf16*>(v_cache), num_slots, m, hq, hkv);
}

int mdb_silu_mul(const void* gate_up, int64_t ld_in, void* act, int64_t ld_act, int m, int inter,
                 mdb_stream_t stream) {
  MDB_REQUIRE(m >= 0 && inter > 0, MDB_ERR_ARG);
  if (m == 0) return MDB_OK;
  MDB_REQUIRE(gate_up && act, MDB_ERR_ARG);
  MDB_REQUIRE(inter % 8 == 0, MDB_ERR_UNSUPPORTED);
  MDB_REQUIRE(ld_in >= 2 * static_cast<int64_t>(inter) && ld_act >= inter, MDB_ERR_ARG);
  MDB_REQUIRE(ld_in % 8 == 0 && ld_act % 8 == 0 && mdb_aligned16(gate_up) && mdb_aligned16(act), MDB_ERR_ALIGN);
  const int64_t total = static_cast<int64_t>(m) * (inter / 8);
  int blocks = static_cast<int>((total + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  return mdb_launch(silu_mul_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const bf16*>(gate_up), ld_in, static_cast<bf16*>(act), ld_act, m, inter);
}

int mdb_gather_rows(const void* table, int64_t num_rows, const int64_t* ids, void* out, int m, int h,
                    mdb_stream_t stream) {
  MDB_REQUIRE(m >= 0 && h > 0 && num_rows > 0, MDB_ERR_ARG);
  if (m == 0) return MDB_OK;
  MDB_REQUIRE(table && ids && out, MDB_ERR_ARG);
  MDB_REQUIRE(h % 8 == 0, MDB_ERR_UNSUPPORTED);
  MDB_REQUIRE(mdb_aligned16(table) && mdb_aligned16(out), MDB_ERR_ALIGN);
  return mdb_launch(gather_rows_kernel, dim3(m), dim3(128), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const bf16*>(table), num_rows, ids, static_cast<bf16*>(out), h);
}

}  // extern "C"
