// One denoising step of the decoder (at most 64 rows) as ONE persistent kernel.
//
// Launched as separate kernels, a 32-row step is bound by the few microseconds
// every kernel costs before and after its work (launch, set-up, first memory
// round trip, completion): 257 launches for 3.4 GB of weights.  Here one CTA
// per SM lives for the whole step.  Its producer thread walks the static list
// of the step's projections (qkv, o, gate/up, down of every layer, LM head)
// and keeps a ring of TMA weight tiles full at all times -- weights depend on
// nothing, so the HBM stream runs straight through the small row phases and
// the grid barriers.  One thread issues tcgen05.mma (weight tile = 128-row A
// operand, the step's rows = narrow B operand, fp32 accumulators in tensor
// memory).  Four worker warps run the epilogues and, between projections,
// the row phases: residual add + RMSNorm, q/k norm + RoPE + KV store, block
// attention over the paged cache (tensor-core flash step), split merge,
// sampler merge.  Phases are separated by a grid barrier (generation counter
// in global memory, bounded spin); activation tiles of a projection are only
// requested once the barrier that completes its input has been passed.
//
// The arithmetic is the device code the stand-alone kernels run (the row sum
// of the RMSNorm is grouped over 128 instead of 256 threads).
//
// Status: correct (tests compare it with the chain of separate kernels), but
// on a 32-row step it is slower than that chain (2.9 ms against 2.0 ms per
// step of the 28-layer decoder): nine dependent phases per layer each cost a
// grid barrier (1.3 - 2 us) and run on only four warps per SM, so the step is
// bound by that latency chain, not by the weight stream.  It is therefore
// off by default (ModelRunner(fused_step=True) or MDB_FUSED_STEP=1 selects it).
#include "mdb_common.cuh"

namespace mdb {

constexpr int kFsThreads = 192;
constexpr int kFsMaxLayers = 64;
constexpr int kFsAttnSmem = kAttnSmemBytes;      // 64 KB: double-buffered K and V tiles

struct FsLayer {
  CUtensorMap map_qkv, map_o, map_gu, map_down;
  const bf16 *ln1, *ln2, *q_norm, *k_norm;
  bf16 *k_cache, *v_cache;
};

struct FsDesc {
  // activation operand maps: x [m,H], attn [m,Hq*D], act [m,I], final [m,H]
  CUtensorMap map_x, map_attn, map_act, map_final, map_lm;
  FsLayer layer[kFsMaxLayers];
  int layers, m, ntok, bs, block, hidden, inter, hq, hkv, vocab;
  int ks_qkv, ks_o, ks_down, nsplit, stages;
  int run_ahead;          // 1: weight tiles are requested before the projection's input is complete
  float eps, scale_log2;
  const bf16* final_ln;
  // buffers
  const bf16* embed_table;
  int64_t embed_rows;
  bf16 *embeds, *x, *res, *q, *attn, *act, *final_rows;
  float* parts;
  float *attn_part_o, *attn_part_ml;
  const float* rope;
  int max_pos;
  // per-step inputs (device buffers the host refreshes before each launch)
  const int64_t* ids;
  const int64_t* positions;
  const int32_t* slots;
  const int32_t* ctx_lens;
  const int32_t* block_table;
  int table_stride, num_pages;
  int64_t num_slots;
  const float* temperatures;
  int noise_mode;
  uint32_t seed;
  const uint32_t* step_dev;
  float4* part_f;
  int* part_i;
  int32_t* x0;
  float* conf;
  unsigned int* grid_bar;   // arrival counter, zeroed by the host before every launch
};

// ---- grid barrier ----------------------------------------------------------------
// Workers only (128 threads, named barrier 1).  One arrival counter in global memory that the host zeroes
// before every launch: barrier k is passed once the counter reaches k * gridDim.x.  Arrival is a single
// release reduction (no round trip), the wait polls with a short back-off and is bounded to 2 s.
__device__ __forceinline__ bool fs_grid_sync(unsigned int* bar, volatile uint32_t* passed_word, uint32_t& passed) {
  bool ok = true;
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (threadIdx.x == 0) {
    const unsigned int target = (passed + 1) * gridDim.x;
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(bar) : "memory");
    unsigned long long deadline = 0;
    for (unsigned int it = 0;; ++it) {
      unsigned int c;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(c) : "l"(bar) : "memory");
      if (c >= target) break;
      __nanosleep(40);
      if ((it & 255u) == 255u) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (deadline == 0) deadline = now + 2000000000ull;
        else if (now > deadline) { ok = false; report_status(MDB_STATUS_WAIT_TIMEOUT); break; }
        if ((*reinterpret_cast<volatile unsigned int*>(&g_device_status) & MDB_STATUS_WAIT_TIMEOUT) != 0) {
          ok = false;   // another wait of this launch already ran out: drain quickly
          break;
        }
      }
    }
    *passed_word = passed + 1;   // the producer reads this to learn which inputs are complete
  }
  ++passed;
  asm volatile("bar.sync 1, 128;" ::: "memory");
  return ok;
}

// ---- row phases run by the 128 worker threads ---------------------------------------

// Residual add + RMSNorm of one row by 128 threads (the arithmetic of add_rmsnorm_kernel).  The input row is
// `xin` (bf16) or the bf16-rounded sum of nparts fp32 slices; red4 is 4 floats of shared memory.
__device__ __noinline__ void fs_norm_row(const bf16* __restrict__ xin, const float* __restrict__ partials,
                                            int nparts, int m, const bf16* __restrict__ residual_in,
                                            const bf16* __restrict__ weight, float eps, bf16* __restrict__ y_out,
                                            bf16* __restrict__ residual_out, int row, int64_t src_row, int h,
                                            float* red4) {
  constexpr int kMaxChunks = 8;   // h <= 128 * 8 * 8 = 8192
  const int chunks = h >> 3;
  const int64_t row_off = static_cast<int64_t>(row) * h;
  float v[kMaxChunks][8];
  float sumsq = 0.f;
#pragma unroll
  for (int it = 0; it < kMaxChunks; ++it) {
    const int c = threadIdx.x + it * 128;
    if (c < chunks) {
      float a[8];
      if (partials != nullptr) {
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = 0.f;
        for (int p = 0; p < nparts; ++p) {
          const float4* src = reinterpret_cast<const float4*>(partials + (static_cast<int64_t>(p) * m + row) * h + c * 8);
          const float4 lo = src[0], hi = src[1];
          a[0] += lo.x; a[1] += lo.y; a[2] += lo.z; a[3] += lo.w;
          a[4] += hi.x; a[5] += hi.y; a[6] += hi.z; a[7] += hi.w;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = bf16_round(a[j]);
      } else {
        const uint4 u = *reinterpret_cast<const uint4*>(xin + src_row * h + c * 8);
        float2 f;
        f = unpack_bf16x2(u.x); a[0] = f.x; a[1] = f.y;
        f = unpack_bf16x2(u.y); a[2] = f.x; a[3] = f.y;
        f = unpack_bf16x2(u.z); a[4] = f.x; a[5] = f.y;
        f = unpack_bf16x2(u.w); a[6] = f.x; a[7] = f.y;
      }
      if (residual_in != nullptr) {
        const uint4 u = *reinterpret_cast<const uint4*>(residual_in + row_off + c * 8);
        float2 f;
        f = unpack_bf16x2(u.x); a[0] += f.x; a[1] += f.y;
        f = unpack_bf16x2(u.y); a[2] += f.x; a[3] += f.y;
        f = unpack_bf16x2(u.z); a[4] += f.x; a[5] += f.y;
        f = unpack_bf16x2(u.w); a[6] += f.x; a[7] += f.y;
      }
      uint4 o;
      o.x = pack_bf16x2(a[0], a[1]); o.y = pack_bf16x2(a[2], a[3]);
      o.z = pack_bf16x2(a[4], a[5]); o.w = pack_bf16x2(a[6], a[7]);
      *reinterpret_cast<uint4*>(residual_out + row_off + c * 8) = o;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[it][j] = a[j];
        sumsq += a[j] * a[j];
      }
    }
  }
  sumsq = warp_sum(sumsq);
  asm volatile("bar.sync 1, 128;" ::: "memory");          // red4 free again
  if ((threadIdx.x & 31) == 0) red4[threadIdx.x >> 5] = sumsq;
  asm volatile("bar.sync 1, 128;" ::: "memory");
  const float total = red4[0] + red4[1] + red4[2] + red4[3];
  const float rstd = 1.0f / sqrtf(total / static_cast<float>(h) + eps);
#pragma unroll
  for (int it = 0; it < kMaxChunks; ++it) {
    const int c = threadIdx.x + it * 128;
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
      for (int j = 0; j < 8; ++j) r[j] = bf16_round(v[it][j] * rstd) * w[j];
      uint4 o;
      o.x = pack_bf16x2(r[0], r[1]); o.y = pack_bf16x2(r[2], r[3]);
      o.z = pack_bf16x2(r[4], r[5]); o.w = pack_bf16x2(r[6], r[7]);
      *reinterpret_cast<uint4*>(y_out + row_off + c * 8) = o;
    }
  }
}

// Sampler merge of one row's partial records by 128 threads (the arithmetic of sampler_finalize_kernel).
__device__ __noinline__ void fs_finalize_row(const float4* __restrict__ part_f, const int* __restrict__ part_i,
                                                int nparts, int m, int row, int32_t* __restrict__ x0_out,
                                                float* __restrict__ conf_out, SampleRec* sh4) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  SampleRec r = {-INFINITY, 0.f, -INFINITY, 0.f, 0x7fffffff};
  for (int p = threadIdx.x; p < nparts; p += 128) {
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
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (lane == 0) sh4[warp] = r;
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (threadIdx.x == 0) {
    SampleRec t = sh4[0];
    for (int w = 1; w < 4; ++w) merge_rec(t, sh4[w]);
    x0_out[row] = t.bi;
    conf_out[row] = expf(t.bl - t.mx) / t.se;
  }
}

// ---- projections ----------------------------------------------------------------------

enum FsEpi { kFsPartial = 0, kFsSwiglu = 1, kFsLmHead = 2 };

struct FsGemm {
  const CUtensorMap* mw;
  const CUtensorMap* mx;
  int tiles, ksplit, chunks_total, chunks_per_slice, epi;
  uint32_t need_bar;      // grid barriers that must have been passed before the activation tiles may be read
  int n;                  // output columns (partial epilogue)
};

// The step's projections in execution order; every role (producer, MMA issue, workers) walks the same list.
__device__ __forceinline__ int fs_num_gemms(const FsDesc& d) { return 4 * d.layers + 1; }

__device__ __forceinline__ FsGemm fs_gemm(const FsDesc& d, int g) {
  FsGemm r;
  const int nqkv = (d.hq + 2 * d.hkv) * kHeadDim;
  if (g == 4 * d.layers) {
    r.mw = &d.map_lm; r.mx = &d.map_final; r.tiles = d.vocab / 128; r.ksplit = 1; r.chunks_total = d.hidden / 64;
    r.epi = kFsLmHead; r.need_bar = 9u * d.layers + 1; r.n = d.vocab;
  } else {
    const int l = g >> 2, w = g & 3;
    const FsLayer& L = d.layer[l];
    if (w == 0) {
      r.mw = &L.map_qkv; r.mx = &d.map_x; r.tiles = nqkv / 128; r.ksplit = d.ks_qkv; r.chunks_total = d.hidden / 64;
      r.epi = kFsPartial; r.need_bar = 9u * l + 1; r.n = nqkv;
    } else if (w == 1) {
      r.mw = &L.map_o; r.mx = &d.map_attn; r.tiles = d.hidden / 128; r.ksplit = d.ks_o;
      r.chunks_total = d.hq * kHeadDim / 64; r.epi = kFsPartial; r.need_bar = 9u * l + 5; r.n = d.hidden;
    } else if (w == 2) {
      r.mw = &L.map_gu; r.mx = &d.map_x; r.tiles = d.inter / 64; r.ksplit = 1; r.chunks_total = d.hidden / 64;
      r.epi = kFsSwiglu; r.need_bar = 9u * l + 7; r.n = 2 * d.inter;
    } else {
      r.mw = &L.map_down; r.mx = &d.map_act; r.tiles = d.hidden / 128; r.ksplit = d.ks_down;
      r.chunks_total = d.inter / 64; r.epi = kFsPartial; r.need_bar = 9u * l + 8; r.n = d.hidden;
    }
  }
  r.chunks_per_slice = (r.chunks_total + r.ksplit - 1) / r.ksplit;
  return r;
}

__device__ __forceinline__ bool fs_aborted() {
  return (*reinterpret_cast<volatile unsigned int*>(&g_device_status) & MDB_STATUS_WAIT_TIMEOUT) != 0;
}

// mbarrier wait bounded to 2 s; leaves at once if any wait of this launch already ran out.  The wait is a
// hardware-suspended try_wait (20 us per attempt), not a spin: the waiting thread shares its scheduler with a
// worker warp and must not take issue slots from it.
__device__ __forceinline__ bool fs_mbar_wait(uint32_t bar, uint32_t parity) {
  unsigned long long deadline = 0;
  for (;;) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(20000u)
        : "memory");
    if (done) return true;
    if (fs_aborted()) return false;
    const unsigned long long now = global_timer_ns();
    if (deadline == 0) deadline = now + kWsWaitLimitNs;
    else if (now > deadline) { report_status(MDB_STATUS_WAIT_TIMEOUT); return false; }
  }
}

// Shared-memory handles the worker functions need.
struct FsSmem {
  uint32_t bar_acc_full, bar_acc_empty, tmem_base, attn_smem;
  float* epi;
};

// Epilogue of every task this CTA owns in projection g (workers only).
__device__ __noinline__ void fs_run_epilogue(const FsDesc& d, int g, const FsSmem sm, int& acc, uint32_t& acc_phase,
                                             uint32_t step) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x;
  const int m = d.m;
  float* epi = sm.epi;
  const uint32_t bar_acc_full = sm.bar_acc_full, bar_acc_empty = sm.bar_acc_empty, tmem_base = sm.tmem_base;

      const FsGemm gm = fs_gemm(d, g);
      const int tasks = gm.tiles * gm.ksplit;
      for (int task = blockIdx.x; task < tasks; task += G) {
        const int tile = task / gm.ksplit, slice = task % gm.ksplit;
        bool ok = fs_mbar_wait(bar_acc_full + 8 * acc, acc_phase);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return;
        tc_fence_after();
        const uint32_t taddr = tmem_base + acc * d.ntok + (static_cast<uint32_t>(32 * warp) << 16);
        float v[64];
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (16 * c < d.ntok) {
            float t16[16];
            tmem_ld16(taddr + 16 * c, t16);
#pragma unroll
            for (int i = 0; i < 16; ++i) v[16 * c + i] = t16[i];
          }
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acc_empty + 8 * acc);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        const int row_local = 32 * warp + lane;
        if (gm.epi == kFsPartial) {
          const int row = tile * kWsTileRows + row_local;
          float* dst = d.parts + static_cast<int64_t>(slice) * m * gm.n + row;
#pragma unroll
          for (int t = 0; t < 64; ++t)
            if (t < m) dst[static_cast<int64_t>(t) * gm.n] = v[t];
        } else if (gm.epi == kFsSwiglu) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            if (half * 32 >= m) break;
#pragma unroll
            for (int t = 0; t < 32; ++t) epi[row_local * 33 + t] = v[32 * half + t];
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int c = threadIdx.x & 63;
            const int tg = threadIdx.x >> 6;
            const int col = tile * 64 + c;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int tt = 16 * tg + i;
              const int r = 32 * half + tt;
              if (r < m) {
                const float gt = bf16_round(epi[c * 33 + tt]);
                const float up = bf16_round(epi[(64 + c) * 33 + tt]);
                const float sl = gt * __frcp_rn(1.0f + __expf(-gt));
                d.act[static_cast<int64_t>(r) * d.inter + col] = __float2bfloat16_rn(bf16_round(sl) * up);
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
          }
        } else {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            if (half * 32 >= m) break;
#pragma unroll
            for (int t = 0; t < 32; ++t) epi[row_local * 33 + t] = v[32 * half + t];
            asm volatile("bar.sync 1, 128;" ::: "memory");
            for (int tt = warp; tt < 32 && 32 * half + tt < m; tt += 4) {
              const int r = 32 * half + tt;
              const float temp = d.temperatures[r / d.block];
              float mx = -INFINITY, bv = -INFINITY, bl = 0.f;
              int bi = 0x7fffffff;
              float lg[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int col = tile * kWsTileRows + lane + 32 * q;
                const float logit = bf16_round(epi[(lane + 32 * q) * 33 + tt]) / temp;
                lg[q] = logit;
                float noisy = logit;
                if (d.noise_mode == 2) noisy += gumbel_noise(d.seed, step, r, col);
                mx = fmaxf(mx, logit);
                if (noisy > bv) { bv = noisy; bl = logit; bi = col; }
              }
              mx = warp_max(mx);
              float se = 0.f;
#pragma unroll
              for (int q = 0; q < 4; ++q) se += expf(lg[q] - mx);
              se = warp_sum(se);
#pragma unroll
              for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const float ol = __shfl_xor_sync(0xffffffffu, bl, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bl = ol; bi = oi; }
              }
              if (lane == 0) {
                d.part_f[static_cast<int64_t>(tile) * m + r] = make_float4(mx, se, bv, bl);
                d.part_i[static_cast<int64_t>(tile) * m + r] = bi;
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
          }
        }
      }
    }

// Block attention items of this CTA for one layer (workers only).
__device__ __noinline__ void fs_attention_phase(const FsDesc& d, const FsLayer& L, uint32_t attn_smem) {
  AttnPagedArgs aa;
  aa.q = d.q; aa.out = d.attn;
  aa.k_cache = L.k_cache; aa.v_cache = L.v_cache;
  aa.block_table = d.block_table; aa.ctx_lens = d.ctx_lens;
  aa.part_o = d.attn_part_o; aa.part_ml = d.attn_part_ml;
  aa.table_stride = d.table_stride; aa.block = d.block; aa.hq = d.hq; aa.hkv = d.hkv;
  aa.num_pages = d.num_pages; aa.nsplit = d.nsplit; aa.scale_log2 = d.scale_log2;
  const int group = d.hq / d.hkv;
  const int row_blocks = (group * d.block + kAttnRows - 1) / kAttnRows;
  const int items = d.bs * d.hkv * row_blocks * d.nsplit;
  for (int it = blockIdx.x; it < items; it += gridDim.x) {
    const int split = it % d.nsplit;
    const int rest = it / d.nsplit;
    const int rb = rest % row_blocks;
    const int kvh = (rest / row_blocks) % d.hkv;
    const int req = rest / (row_blocks * d.hkv);
    attn_paged_item<true>(aa, attn_smem, split, kvh, rb, req);
    asm volatile("bar.sync 1, 128;" ::: "memory");
  }
}

// ---- the kernel --------------------------------------------------------------------------
__global__ void __launch_bounds__(kFsThreads, 1)
fused_step_kernel(const FsDesc* __restrict__ dp) {
  const FsDesc& d = *dp;
  extern __shared__ unsigned char fs_smem_raw[];
  const uint32_t raw = smem_u32(fs_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* gen_base = fs_smem_raw + (base - raw);
  const int stages = d.stages;
  const int x_tile_bytes = d.ntok * kWsBK * 2;
  const uint32_t w_tiles = base;
  const uint32_t x_tiles = w_tiles + stages * kWsWTileBytes;
  const uint32_t attn_off = stages * (kWsWTileBytes + x_tile_bytes);
  const uint32_t attn_smem = base + attn_off;
  const uint32_t epi_off = attn_off + kFsAttnSmem;
  float* epi = reinterpret_cast<float*>(gen_base + epi_off);
  const uint32_t bars_off = epi_off + kWsEpiFloats * 4;
  const uint32_t bars = base + bars_off;
  const uint32_t bar_full = bars, bar_empty = bars + 8 * stages;
  const uint32_t bar_acc_full = bars + 16 * stages, bar_acc_empty = bar_acc_full + 16;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(gen_base + bars_off + 16 * stages + 32);
  // misc[0] = tensor-memory base, misc[1] = grid barriers passed by this CTA's workers
  float* red4 = reinterpret_cast<float*>(gen_base + bars_off + 16 * stages + 32 + 16);
  SampleRec* sh4 = reinterpret_cast<SampleRec*>(gen_base + bars_off + 16 * stages + 32 + 32);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tmem_cols = 2 * d.ntok <= 32 ? 32 : (2 * d.ntok <= 64 ? 64 : 128);
  const int G = gridDim.x;
  const int ngemm = fs_num_gemms(d);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 4);
    }
    misc[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    const uint32_t slot = smem_u32(const_cast<uint32_t*>(&misc[0]));
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = misc[0];

  if (warp == 4) {
    // =============== producer: weight tiles always, activation tiles once their input is complete ===============
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      // activation tiles not yet requested: ring position, map, k column, barrier count they need
      int def_n = 0, def_stage0 = 0;
      const CUtensorMap* def_map[16];
      int def_k[16];
      uint32_t def_need[16];
      bool ok = true;
      // Request the pending activation tiles whose input is complete, oldest first.  With `force` the oldest one
      // is waited for (bounded): the ring is full and nothing can move until it is requested.
      auto flush = [&](bool force) {
        int done = 0;
        while (done < def_n && ok) {
          if (misc[1] < def_need[done]) {
            if (!force || done > 0) break;
            unsigned long long deadline = 0;
            for (uint32_t it = 0; misc[1] < def_need[done]; ++it) {
              __nanosleep(500);
              if ((it & 255u) == 255u) {
                if (fs_aborted()) { ok = false; break; }
                const unsigned long long now = global_timer_ns();
                if (deadline == 0) deadline = now + kWsWaitLimitNs;
                else if (now > deadline) { report_status(MDB_STATUS_WAIT_TIMEOUT); ok = false; break; }
              }
            }
            if (!ok) break;
          }
          // the workers' global stores were published by the grid barrier; order them before the async-proxy read
          asm volatile("fence.proxy.async.global;" ::: "memory");
          const int s = (def_stage0 + done) % stages;
          tma_load_2d(x_tiles + s * x_tile_bytes, def_map[done], def_k[done], 0, bar_full + 8 * s);
          ++done;
        }
        if (done > 0) {
          for (int i = done; i < def_n; ++i) {
            def_map[i - done] = def_map[i]; def_k[i - done] = def_k[i]; def_need[i - done] = def_need[i];
          }
          def_n -= done;
          def_stage0 = (def_stage0 + done) % stages;
        }
      };
      for (int g = 0; g < ngemm && ok; ++g) {
        const FsGemm gm = fs_gemm(d, g);
        const int tasks = gm.tiles * gm.ksplit;
        if (!d.run_ahead) {
          for (uint32_t it = 0; misc[1] < gm.need_bar && it < (1u << 24); ++it) __nanosleep(100);
        }
        for (int task = blockIdx.x; task < tasks && ok; task += G) {
          const int tile = task / gm.ksplit, slice = task % gm.ksplit;
          const int chunk0 = slice * gm.chunks_per_slice;
          const int nchunks = min(gm.chunks_per_slice, gm.chunks_total - chunk0);
          for (int c = 0; c < nchunks; ++c) {
            if (def_n == stages) flush(true);   // the ring is full of tiles that wait for activations
            if (!ok) break;
            if (!fs_mbar_wait(bar_empty + 8 * stage, phase ^ 1)) { ok = false; break; }
            const int kcol = (chunk0 + c) * kWsBK;
            const uint32_t full = bar_full + 8 * stage;
            mbar_arrive_expect_tx(full, kWsWTileBytes + x_tile_bytes);
            const uint32_t wdst = w_tiles + stage * kWsWTileBytes;
            if (gm.epi == kFsSwiglu) {
              tma_load_2d(wdst, gm.mw, kcol, tile * 64, full);
              tma_load_2d(wdst + kWsWTileBytes / 2, gm.mw, kcol, d.inter + tile * 64, full);
            } else {
              tma_load_2d(wdst, gm.mw, kcol, tile * kWsTileRows, full);
            }
            if (def_n == 0 && misc[1] >= gm.need_bar) {
              asm volatile("fence.proxy.async.global;" ::: "memory");
              tma_load_2d(x_tiles + stage * x_tile_bytes, gm.mx, kcol, 0, full);
            } else {
              if (def_n == 0) def_stage0 = stage;
              def_map[def_n] = gm.mx; def_k[def_n] = kcol; def_need[def_n] = gm.need_bar;
              ++def_n;
            }
            if (++stage == stages) { stage = 0; phase ^= 1; }
            // opportunistic: request pending activation tiles as soon as their barrier has been passed
            if (def_n > 0 && misc[1] >= def_need[0]) flush(false);
          }
        }
      }
      while (ok && def_n > 0) flush(true);
    }
  } else if (warp == 5) {
    // =============== MMA issue ===============
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(d.ntok);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int g = 0; g < ngemm && ok; ++g) {
        const FsGemm gm = fs_gemm(d, g);
        const int tasks = gm.tiles * gm.ksplit;
        for (int task = blockIdx.x; task < tasks && ok; task += G) {
          const int chunk0 = (task % gm.ksplit) * gm.chunks_per_slice;
          const int nchunks = min(gm.chunks_per_slice, gm.chunks_total - chunk0);
          if (!fs_mbar_wait(bar_acc_empty + 8 * acc, acc_phase ^ 1)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * d.ntok;
          for (int c = 0; c < nchunks; ++c) {
            if (!fs_mbar_wait(bar_full + 8 * stage, phase)) { ok = false; break; }
            tc_fence_after();
            const uint64_t adesc = umma_desc_sw128(w_tiles + stage * kWsWTileBytes);
            const uint64_t bdesc = umma_desc_sw128(x_tiles + stage * x_tile_bytes);
#pragma unroll
            for (int k16 = 0; k16 < kWsBK / 16; ++k16)
              umma_bf16(d_tmem, adesc + 2 * k16, bdesc + 2 * k16, idesc, (c > 0 || k16 > 0) ? 1u : 0u);
            umma_commit(bar_empty + 8 * stage);
            if (++stage == stages) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          umma_commit(bar_acc_full + 8 * acc);
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
      }
    }
  } else {
    // =============== workers: row phases and epilogues ===============
    uint32_t passed = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    const int nqkv = (d.hq + 2 * d.hkv) * kHeadDim;
    const int nheads = d.hq + 2 * d.hkv;
    const int h = d.hidden;
    const int m = d.m;
    const uint32_t step = (d.noise_mode == 2 && d.step_dev != nullptr) ? *d.step_dev : 0u;

    FsSmem sm;
    sm.bar_acc_full = bar_acc_full; sm.bar_acc_empty = bar_acc_empty; sm.tmem_base = tmem_base;
    sm.attn_smem = attn_smem; sm.epi = epi;
    int tr = 0;
    for (int l = 0; l < d.layers; ++l) {
      const FsLayer& L = d.layer[l];
      tr = 0;
      // input RMSNorm: layer 0 reads the embedding rows of the step's ids, later layers the down projection's slices
      for (int row = blockIdx.x; row < m; row += G) {
        if (l == 0) {
          int64_t id = d.ids[row];
          if (id < 0 || id >= d.embed_rows) { if (threadIdx.x == 0) report_status(MDB_STATUS_BAD_TOKEN); id = 0; }
          fs_norm_row(d.embed_table, nullptr, 0, m, nullptr, L.ln1, d.eps, d.x, d.res, row, id, h, red4);
        } else {
          fs_norm_row(nullptr, d.parts, d.ks_down, m, d.res, L.ln1, d.eps, d.x, d.res, row, row, h, red4);
        }
      }
      if (l == 1 && threadIdx.x == 0) trace_event(20, 100 + tr);
      fs_grid_sync(d.grid_bar, &misc[1], passed);
      if (l == 1 && threadIdx.x == 0) trace_event(20, tr); ++tr;
      fs_run_epilogue(d, 4 * l + 0, sm, acc, acc_phase, step);                                                 // qkv slices
      if (l == 1 && threadIdx.x == 0) trace_event(20, 100 + tr);
      fs_grid_sync(d.grid_bar, &misc[1], passed);
      if (l == 1 && threadIdx.x == 0) trace_event(20, tr); ++tr;
      for (int w = blockIdx.x * 4 + warp; w < m * nheads; w += G * 4)          // q/k norm, RoPE, KV store
        qknorm_rope_commit_warp(w / nheads, w % nheads, lane, nullptr, 0, d.parts, d.ks_qkv, d.positions, d.rope,
                                d.max_pos, L.q_norm, L.k_norm, d.eps, d.slots, d.q, nullptr, nullptr, L.k_cache,
                                L.v_cache, d.num_slots, m, d.hq, d.hkv);
      if (l == 1 && threadIdx.x == 0) trace_event(20, 100 + tr);
      fs_grid_sync(d.grid_bar, &misc[1], passed);
      if (l == 1 && threadIdx.x == 0) trace_event(20, tr); ++tr;
      fs_attention_phase(d, L, attn_smem);                                      // block attention over the paged cache
      if (l == 1 && threadIdx.x == 0) trace_event(20, 100 + tr);
      fs_grid_sync(d.grid_bar, &misc[1], passed);
      if (l == 1 && threadIdx.x == 0) trace_event(20, tr); ++tr;
      if (d.nsplit > 1)
        for (int w = blockIdx.x * 4 + warp; w < d.bs * d.hq * d.block; w += G * 4)
          attn_combine_row(d.attn_part_o, d.attn_part_ml, d.attn, d.block, d.hq, d.nsplit, w, lane);
      if (l == 1 && threadIdx.x == 0) trace_event(20, 100 + tr);
      fs_grid_sync(d.grid_bar, &misc[1], passed);
      if (l == 1 && threadIdx.x == 0) trace_event(20, tr); ++tr;
      fs_run_epilogue(d, 4 * l + 1, sm, acc, acc_phase, step);                                                 // o_proj slices
      if (l == 1 && threadIdx.x == 0) trace_event(20, 100 + tr);
      fs_grid_sync(d.grid_bar, &misc[1], passed);
      if (l == 1 && threadIdx.x == 0) trace_event(20, tr); ++tr;
      for (int row = blockIdx.x; row < m; row += G)
        fs_norm_row(nullptr, d.parts, d.ks_o, m, d.res, L.ln2, d.eps, d.x, d.res, row, row, h, red4);
      if (l == 1 && threadIdx.x == 0) trace_event(20, 100 + tr);
      fs_grid_sync(d.grid_bar, &misc[1], passed);
      if (l == 1 && threadIdx.x == 0) trace_event(20, tr); ++tr;
      fs_run_epilogue(d, 4 * l + 2, sm, acc, acc_phase, step);                                                 // gate/up + SiLU*mul
      if (l == 1 && threadIdx.x == 0) trace_event(20, 100 + tr);
      fs_grid_sync(d.grid_bar, &misc[1], passed);
      if (l == 1 && threadIdx.x == 0) trace_event(20, tr); ++tr;
      fs_run_epilogue(d, 4 * l + 3, sm, acc, acc_phase, step);                                                 // down_proj slices
      if (l == 1 && threadIdx.x == 0) trace_event(20, 100 + tr);
      fs_grid_sync(d.grid_bar, &misc[1], passed);
      if (l == 1 && threadIdx.x == 0) trace_event(20, tr); ++tr;
    }
    for (int row = blockIdx.x; row < m; row += G)
      fs_norm_row(nullptr, d.parts, d.ks_down, m, d.res, d.final_ln, d.eps, d.final_rows, d.res, row, row, h, red4);
    fs_grid_sync(d.grid_bar, &misc[1], passed);
    fs_run_epilogue(d, 4 * d.layers, sm, acc, acc_phase, step);                                                // LM head scan
    fs_grid_sync(d.grid_bar, &misc[1], passed);
    for (int row = blockIdx.x; row < m; row += G)
      fs_finalize_row(d.part_f, d.part_i, d.vocab / kWsTileRows, m, row, d.x0, d.conf, sh4);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

struct LmHeadLayoutFs {
  int64_t off_i;
};
// offsets of the sampler records inside the LM-head workspace (same as the stand-alone LM head for m <= 64)
static LmHeadLayoutFs lmhead_layout_fs(int m, int vocab) {
  const int64_t nparts = (vocab + 31) / 32;
  LmHeadLayoutFs l;
  l.off_i = (nparts * m * 16 + 255) / 256 * 256;
  return l;
}

static int fs_smem_bytes(int stages, int ntok) {
  return 1024 + stages * (kWsWTileBytes + ntok * kWsBK * 2) + kFsAttnSmem + kWsEpiFloats * 4 + 16 * stages + 32 + 16 +
         16 + 4 * static_cast<int>(sizeof(SampleRec)) + 16;
}

}  // namespace mdb

using namespace mdb;

extern "C" {

int64_t mdb_fused_step_desc_bytes(void) { return static_cast<int64_t>(sizeof(FsDesc)); }

int mdb_fused_step_create(const mdb_fused_step_params* p, void* desc_device) {
  MDB_REQUIRE(p != nullptr && desc_device != nullptr, MDB_ERR_ARG);
  MDB_REQUIRE(p->layers >= 1 && p->layers <= kFsMaxLayers && p->m >= 1 && p->m <= 64 && p->bs >= 1, MDB_ERR_UNSUPPORTED);
  MDB_REQUIRE(p->bs * p->block == p->m, MDB_ERR_ARG);
  const int nqkv = (p->hq + 2 * p->hkv) * kHeadDim;
  MDB_REQUIRE(p->hidden % 128 == 0 && p->hidden <= 8192 && nqkv % 128 == 0 && p->inter % 64 == 0 &&
                  p->vocab % 128 == 0 && p->hq % p->hkv == 0,
              MDB_ERR_UNSUPPORTED);
  MDB_REQUIRE(p->noise_mode == 0 || p->noise_mode == 2, MDB_ERR_UNSUPPORTED);
  MDB_REQUIRE(p->ks_qkv >= 1 && p->ks_o >= 1 && p->ks_down >= 1 && p->nsplit >= 1, MDB_ERR_ARG);
  MDB_REQUIRE(p->w_qkv && p->w_o && p->w_gate_up && p->w_down && p->ln1 && p->ln2 && p->q_norm && p->k_norm &&
                  p->k_cache && p->v_cache && p->final_ln && p->embed_table && p->lm_head && p->x && p->res && p->q &&
                  p->attn && p->act && p->final_rows && p->parts && p->rope && p->ids && p->positions && p->slots &&
                  p->ctx_lens && p->block_table && p->temperatures && p->lm_ws && p->x0 && p->conf && p->grid_bar,
              MDB_ERR_ARG);
  MDB_REQUIRE(p->nsplit == 1 || p->attn_ws != nullptr, MDB_ERR_ARG);
  FsDesc* d = new FsDesc();
  memset(d, 0, sizeof(FsDesc));
  const int ntok = (p->m + 15) / 16 * 16;
  bool ok = true;
  ok = ok && get_tensor_map(p->x, p->m, p->hidden, p->hidden, ntok, &d->map_x);
  ok = ok && get_tensor_map(p->attn, p->m, p->hq * kHeadDim, p->hq * kHeadDim, ntok, &d->map_attn);
  ok = ok && get_tensor_map(p->act, p->m, p->inter, p->inter, ntok, &d->map_act);
  ok = ok && get_tensor_map(p->final_rows, p->m, p->hidden, p->hidden, ntok, &d->map_final);
  ok = ok && get_tensor_map(p->lm_head, p->vocab, p->hidden, p->hidden, kWsTileRows, &d->map_lm);
  for (int l = 0; l < p->layers && ok; ++l) {
    FsLayer& L = d->layer[l];
    ok = ok && get_tensor_map(p->w_qkv[l], nqkv, p->hidden, p->hidden, kWsTileRows, &L.map_qkv);
    ok = ok && get_tensor_map(p->w_o[l], p->hidden, p->hq * kHeadDim, p->hq * kHeadDim, kWsTileRows, &L.map_o);
    ok = ok && get_tensor_map(p->w_gate_up[l], 2 * p->inter, p->hidden, p->hidden, 64, &L.map_gu);
    ok = ok && get_tensor_map(p->w_down[l], p->hidden, p->inter, p->inter, kWsTileRows, &L.map_down);
    L.ln1 = static_cast<const bf16*>(p->ln1[l]);
    L.ln2 = static_cast<const bf16*>(p->ln2[l]);
    L.q_norm = static_cast<const bf16*>(p->q_norm[l]);
    L.k_norm = static_cast<const bf16*>(p->k_norm[l]);
    L.k_cache = static_cast<bf16*>(p->k_cache[l]);
    L.v_cache = static_cast<bf16*>(p->v_cache[l]);
  }
  if (!ok) { delete d; return MDB_ERR_CUDA; }
  d->layers = p->layers; d->m = p->m; d->ntok = ntok; d->bs = p->bs; d->block = p->block; d->hidden = p->hidden;
  d->inter = p->inter; d->hq = p->hq; d->hkv = p->hkv; d->vocab = p->vocab;
  d->ks_qkv = p->ks_qkv; d->ks_o = p->ks_o; d->ks_down = p->ks_down; d->nsplit = p->nsplit;
  int stages = 12;
  while (stages > 2 && fs_smem_bytes(stages, ntok) > 227 * 1024) --stages;
  d->stages = stages;
  d->run_ahead = 1;
  d->eps = p->eps;
  d->scale_log2 = p->softmax_scale * 1.4426950408889634f;
  d->final_ln = static_cast<const bf16*>(p->final_ln);
  d->embed_table = static_cast<const bf16*>(p->embed_table);
  d->embed_rows = p->embed_rows;
  d->x = static_cast<bf16*>(p->x); d->res = static_cast<bf16*>(p->res); d->q = static_cast<bf16*>(p->q);
  d->attn = static_cast<bf16*>(p->attn); d->act = static_cast<bf16*>(p->act);
  d->final_rows = static_cast<bf16*>(p->final_rows);
  d->parts = p->parts;
  d->attn_part_o = static_cast<float*>(p->attn_ws);
  d->attn_part_ml = d->attn_part_o ? d->attn_part_o + static_cast<int64_t>(p->bs) * p->nsplit * p->hq * p->block * kHeadDim
                                   : nullptr;
  d->rope = p->rope; d->max_pos = p->max_pos;
  d->ids = p->ids; d->positions = p->positions; d->slots = p->slots; d->ctx_lens = p->ctx_lens;
  d->block_table = p->block_table; d->table_stride = p->table_stride; d->num_pages = p->num_pages;
  d->num_slots = p->num_slots;
  d->temperatures = p->temperatures; d->noise_mode = p->noise_mode; d->seed = p->seed; d->step_dev = p->step_dev;
  // LM-head records: same layout as mdb_lmhead_sample's workspace
  const LmHeadLayoutFs lay = lmhead_layout_fs(p->m, p->vocab);
  d->part_f = reinterpret_cast<float4*>(p->lm_ws);
  d->part_i = reinterpret_cast<int*>(static_cast<unsigned char*>(p->lm_ws) + lay.off_i);
  d->x0 = p->x0; d->conf = p->conf; d->grid_bar = p->grid_bar;
  const cudaError_t e = cudaMemcpy(desc_device, d, sizeof(FsDesc), cudaMemcpyHostToDevice);
  delete d;
  return e == cudaSuccess ? MDB_OK : MDB_ERR_CUDA;
}

int mdb_fused_step_launch(const void* desc_device, uint32_t* grid_bar, int m, mdb_stream_t stream) {
  MDB_REQUIRE(desc_device != nullptr && grid_bar != nullptr && m >= 1 && m <= 64, MDB_ERR_ARG);
  static int sm_count = 0;
  const int ntok = (m + 15) / 16 * 16;
  int stages = 12;
  while (stages > 2 && fs_smem_bytes(stages, ntok) > 227 * 1024) --stages;
  const int smem = fs_smem_bytes(stages, ntok);
  if (sm_count == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return MDB_ERR_CUDA;
    if (cudaFuncSetAttribute(fused_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
      return MDB_ERR_CUDA;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fused_step_kernel, kFsThreads, 227 * 1024) !=
            cudaSuccess || per_sm < 1)
      return MDB_ERR_UNSUPPORTED;
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) return MDB_ERR_CUDA;
  }
  // every CTA must be resident at once: the phases meet at grid barriers
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sm_count);
  cfg.blockDim = dim3(kFsThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const FsDesc* dp = static_cast<const FsDesc*>(desc_device);
  if (cudaMemsetAsync(grid_bar, 0, 4, cfg.stream) != cudaSuccess) return MDB_ERR_CUDA;
  return cudaLaunchKernelEx(&cfg, fused_step_kernel, dp) == cudaSuccess ? MDB_OK : MDB_ERR_CUDA;
}

}  // extern "C"
