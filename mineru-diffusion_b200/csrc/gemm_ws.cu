// Weight-streaming linear layers on the 5th-generation tensor cores.
//
// For a denoising step of at most 64 rows each projection reads its weight
// once and is bound by HBM.  The kernel is built so that the weight stream
// never stops: a persistent CTA per SM, one producer thread issuing TMA tile
// loads (128 weight rows x 64 k, 128-byte swizzle) into a ring of up to ten
// shared-memory stages (200 KB in flight per SM), one thread issuing
// tcgen05.mma with the WEIGHT tile as the 128-row A operand and the step's
// activations as the narrow B operand (N = rows of the step, 16..64), fp32
// accumulators in tensor memory (two buffers, so the epilogue of one tile
// overlaps the stream of the next), and four epilogue warps that read the
// accumulators with tcgen05.ld -- one weight row per thread, one activation
// row per register.
//
// Launched with programmatic dependent launch, the producer starts streaming
// weights (which no earlier kernel writes) before the preceding kernel has
// finished, and only waits for it before loading activations or storing.
//
// Work unit: (tile of 128 weight rows, k slice).  Epilogues: fp32 split-k
// slice; bf16 store; SiLU(gate)*up for a tile made of 64 gate rows and their
// 64 up rows; LM-head scan (temperature, Gumbel noise, max / sum-exp /
// argmax per step row) that never writes a logit.
//
// Every wait on an mbarrier is bounded; on expiry the CTA raises
// MDB_STATUS_WAIT_TIMEOUT, stops issuing work, and leaves after freeing its
// tensor memory.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "mdb_common.cuh"

namespace mdb {

enum WsEpilogue { kWsPartial = 0, kWsBf16 = 1, kWsSwiglu = 2, kWsLmHead = 3 };

constexpr int kWsTileRows = 128;          // weight rows per tile = UMMA M
constexpr int kWsBK = 64;                 // k per stage: one 128-byte swizzle atom of bf16
constexpr int kWsWTileBytes = kWsTileRows * kWsBK * 2;   // 16 KB
constexpr int kWsThreads = 192;           // warps 0-3 epilogue, 4 producer, 5 MMA
constexpr int kWsMaxRows = 64;            // step rows of the fused epilogues (bf16, SiLU*mul, LM head)
constexpr int kWsMaxRowsPartial = 256;    // step rows of the split-k slice form = the widest UMMA N
constexpr int kWsEpiFloats = kWsTileRows * 33;           // staging tile [128][33] fp32

struct WsArgs {
  int m, n, k;
  int ntok;            // activation rows padded to a multiple of 16 (UMMA N)
  int tiles_n;         // weight-row tiles
  int ksplit;          // k slices
  int chunks_per_slice;  // 64-wide k chunks per slice (last slice may be shorter)
  int chunks_total;    // k / 64
  int stages;
  int inter;           // swiglu: rows of the gate half
  float* partials;     // [ksplit][m][n]
  bf16* y;             // bf16 / swiglu output
  int64_t ldy;
  const float* temperatures;
  int block;
  int noise_mode;
  const float* noise;
  uint32_t seed, step;
  const uint32_t* step_dev;
  float4* part_f;      // [tiles_total][m]
  int* part_i;
  // tensor-parallel pair (all null / zero on one GPU)
  int tile_begin;            // first weight-row tile this rank owns (LM head: vocabulary shard)
  int tiles_override;        // > 0: number of tiles this rank processes instead of all of them
  float* peer_partials;      // same layout as partials, in the peer's memory
  float4* peer_part_f;       // LM head records mirrored into the peer's memory
  int* peer_part_i;
  TpSignal tp;
};

// ---- PTX wrappers ------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait for the phase with the given parity; false once the wait limit (2 s by default: far beyond any
// legitimate wait of a decode step) has passed.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  unsigned long long deadline = 0;
  for (uint32_t it = 0;; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if ((it & 1023u) == 1023u) {
      const unsigned long long now = global_timer_ns();
      if (deadline == 0) deadline = now + g_wait_limit_ns;
      else if (now > deadline) return false;
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);        // start address / 16
  d |= static_cast<uint64_t>(1) << 16;                          // leading byte offset / 16 (unused for swizzled K-major)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                  // stride byte offset / 16
  d |= static_cast<uint64_t>(1) << 46;                          // descriptor version of this architecture
  d |= static_cast<uint64_t>(2) << 61;                          // 128-byte swizzle
  return d;
}
// bf16 x bf16 -> fp32, both operands K-major, M = 128, N = ntok
__device__ __forceinline__ uint32_t umma_idesc_bf16(int ntok) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(ntok >> 3) << 17) |
         (static_cast<uint32_t>(kWsTileRows >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 16 consecutive fp32 columns
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- warp-collective forms --------------------------------------------------
// Every lane of a converged warp makes the call with the same arguments and one elected lane issues the
// instruction.  With the operands warp-uniform the compiler keeps descriptors, coordinates and barrier
// addresses in the uniform datapath the TMA and tcgen05 instructions read from; issued from a single
// divergent lane instead, each tcgen05.mma costs ~165 cycles and each TMA tile load ~115 cycles of issue
// time (measured), against ~50 and ~27 this way -- enough to make small-N MMAs issue-bound.
__device__ __forceinline__ bool mbar_wait_w(uint32_t bar, uint32_t parity) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity)) != 0;
}
__device__ __forceinline__ void mbar_arrive_expect_tx_w(uint32_t bar, uint32_t bytes) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t}"
      ::"r"(bar), "r"(bytes)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_w(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n\t}"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_w(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit_w(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(bar)
      : "memory");
}

// ---- kernel ------------------------------------------------------------------
template <int EPI>
__global__ void __launch_bounds__(kWsThreads, 1)
gemm_ws_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const WsArgs a) {
  extern __shared__ unsigned char ws_smem_raw[];
  // carve: [stages x W tile][stages x X tile][epilogue staging][barriers]
  const uint32_t raw = smem_u32(ws_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* gen_base = ws_smem_raw + (base - raw);
  const int x_tile_bytes = a.ntok * kWsBK * 2;
  const uint32_t w_tiles = base;
  const uint32_t x_tiles = w_tiles + a.stages * kWsWTileBytes;
  const uint32_t epi_off = a.stages * (kWsWTileBytes + x_tile_bytes);
  float* epi = reinterpret_cast<float*>(gen_base + epi_off);
  const uint32_t bars = base + epi_off + kWsEpiFloats * 4;
  // barrier slots (8 bytes each): full[stages], empty[stages], acc_full[2], acc_empty[2]; then tmem base, abort flag
  const uint32_t bar_full = bars, bar_empty = bars + 8 * a.stages;
  const uint32_t bar_acc_full = bars + 16 * a.stages, bar_acc_empty = bar_acc_full + 16;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(gen_base + epi_off + kWsEpiFloats * 4 + 16 * a.stages + 32);
  // misc[0] = tensor-memory base address, misc[1] = abort flag

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tasks = a.tiles_n * a.ksplit;
  if (threadIdx.x == 0) trace_event(EPI, 0);
  uint32_t tmem_cols = 32;          // two accumulator buffers of ntok columns, rounded up to a power of two
  while (tmem_cols < 2u * a.ntok) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
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
  pdl_launch_dependents();
  if (threadIdx.x == 0) trace_event(EPI, 1);

  auto task_tile = [&](int task) { return a.tile_begin + task / a.ksplit; };
  auto task_slice = [&](int task) { return task % a.ksplit; };
  auto slice_chunks = [&](int slice) {
    const int beg = slice * a.chunks_per_slice;
    return min(a.chunks_per_slice, a.chunks_total - beg);
  };

  if (warp == 4) {
    // ---------------- producer: TMA loads ----------------
    // The whole warp walks the loop with warp-uniform operands; one elected lane issues each instruction.
    int stage = 0;
    uint32_t phase = 0;
    bool deps_ready = false;
    int deferred = 0;             // leading chunks (stage d for chunk d) whose activation tile is still to be issued
    bool ok = true;
    // k column of the d-th chunk this CTA processes
    auto kcol_of = [&](int d) {
      for (int task = blockIdx.x; task < tasks; task += gridDim.x) {
        const int slice = task_slice(task);
        const int n = slice_chunks(slice);
        if (d < n) return (slice * a.chunks_per_slice + d) * kWsBK;
        d -= n;
      }
      return 0;
    };
    auto flush_deferred = [&]() {
      if (lane == 0) trace_event(EPI, 2);
      pdl_wait();
      if (lane == 0) trace_event(EPI, 3);
      deps_ready = true;
      for (int d = 0; d < deferred; ++d)
        tma_load_2d_w(x_tiles + d * x_tile_bytes, &map_x, kcol_of(d), 0, bar_full + 8 * d);
      deferred = 0;
    };
    for (int task = blockIdx.x; task < tasks && ok; task += gridDim.x) {
      const int tile = task_tile(task), slice = task_slice(task);
      const int nchunks = slice_chunks(slice);
      const int chunk0 = slice * a.chunks_per_slice;
      for (int c = 0; c < nchunks; ++c) {
        // ring full of weight tiles: now the activations are needed
        if (!deps_ready && deferred == a.stages) flush_deferred();
        if (!mbar_wait_w(bar_empty + 8 * stage, phase ^ 1)) { ok = false; break; }
        const int kcol = (chunk0 + c) * kWsBK;
        const uint32_t full = bar_full + 8 * stage;
        mbar_arrive_expect_tx_w(full, kWsWTileBytes + x_tile_bytes);
        const uint32_t wdst = w_tiles + stage * kWsWTileBytes;
        if (EPI == kWsSwiglu) {
          tma_load_2d_w(wdst, &map_w, kcol, tile * 64, full);                       // 64 gate rows
          tma_load_2d_w(wdst + kWsWTileBytes / 2, &map_w, kcol, a.inter + tile * 64, full);   // their up rows
        } else {
          tma_load_2d_w(wdst, &map_w, kcol, tile * kWsTileRows, full);
        }
        if (deps_ready) tma_load_2d_w(x_tiles + stage * x_tile_bytes, &map_x, kcol, 0, full);
        else ++deferred;          // the first chunks sit in stages 0, 1, ... in order
        if (++stage == a.stages) { stage = 0; phase ^= 1; }
      }
    }
    if (!deps_ready) flush_deferred();
    if (!ok && lane == 0) { misc[1] = 1; report_status(MDB_STATUS_WAIT_TIMEOUT); }
  } else if (warp == 5) {
    // ---------------- MMA issue (warp-collective, see above) ----------------
    const uint32_t idesc = umma_idesc_bf16(a.ntok);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int task = blockIdx.x; task < tasks && ok; task += gridDim.x) {
      const int nchunks = slice_chunks(task_slice(task));
      if (!mbar_wait_w(bar_acc_empty + 8 * acc, acc_phase ^ 1)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * a.ntok;
      for (int c = 0; c < nchunks; ++c) {
        if (!mbar_wait_w(bar_full + 8 * stage, phase)) { ok = false; break; }
        if (c == 0 && lane == 0) trace_event(EPI, 4);
        tc_fence_after();
        const uint64_t adesc = umma_desc_sw128(w_tiles + stage * kWsWTileBytes);
        const uint64_t bdesc = umma_desc_sw128(x_tiles + stage * x_tile_bytes);
#pragma unroll
        for (int k16 = 0; k16 < kWsBK / 16; ++k16)   // 32 bytes further along k inside the swizzle atom
          umma_bf16_w(d_tmem, adesc + 2 * k16, bdesc + 2 * k16, idesc, (c > 0 || k16 > 0) ? 1u : 0u);
        umma_commit_w(bar_empty + 8 * stage);          // stage reusable once these MMAs have read it
        if (++stage == a.stages) { stage = 0; phase ^= 1; }
      }
      if (!ok) break;
      umma_commit_w(bar_acc_full + 8 * acc);           // accumulator complete
      if (lane == 0) trace_event(EPI, 5);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (!ok && lane == 0) { misc[1] = 1; report_status(MDB_STATUS_WAIT_TIMEOUT); }
  } else {
    // ---------------- epilogue warps 0..3: tensor-memory lanes 32*warp .. +31 ----------------
    int acc = 0;
    uint32_t acc_phase = 0;
    bool waited_deps = false;
    uint32_t step = a.step;
    for (int task = blockIdx.x; task < tasks; task += gridDim.x) {
      const int tile = task_tile(task), slice = task_slice(task);
      bool ok = mbar_wait(bar_acc_full + 8 * acc, acc_phase);
      ok = __all_sync(0xffffffffu, ok) && misc[1] == 0;
      if (!ok) {
        if (lane == 0) { misc[1] = 1; report_status(MDB_STATUS_WAIT_TIMEOUT); }
        break;
      }
      if (threadIdx.x == 0) trace_event(EPI, 6);
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * a.ntok + (static_cast<uint32_t>(32 * warp) << 16);
      if (EPI == kWsPartial && a.ntok > 64) {
        // more than 64 step rows: the accumulator row of a thread is drained 64 columns at a time
        const int row = tile * kWsTileRows + 32 * warp + lane;
        float* dst = a.partials + static_cast<int64_t>(slice) * a.m * a.n + row;
        for (int t0 = 0; t0 < a.ntok; t0 += 64) {
          float v[64];
#pragma unroll
          for (int c = 0; c < 4; ++c)
            if (t0 + 16 * c < a.ntok) {
              float t16[16];
              tmem_ld16(taddr + t0 + 16 * c, t16);
#pragma unroll
              for (int i = 0; i < 16; ++i) v[16 * c + i] = t16[i];
            }
          tmem_ld_wait();
          if (t0 + 64 >= a.ntok) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + 8 * acc);   // accumulator buffer may be overwritten
          }
          if (!waited_deps) {
            pdl_wait();
            waited_deps = true;
          }
#pragma unroll
          for (int t = 0; t < 64; ++t)
            if (t0 + t < a.m) dst[static_cast<int64_t>(t0 + t) * a.n] = v[t];
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        continue;
      }
      float v[64];
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (16 * c < a.ntok) {
          float t16[16];
          tmem_ld16(taddr + 16 * c, t16);
#pragma unroll
          for (int i = 0; i < 16; ++i) v[16 * c + i] = t16[i];
        }
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * acc);   // accumulator buffer may be overwritten
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      if (!waited_deps) {
        pdl_wait();
        waited_deps = true;
        if (EPI == kWsLmHead && a.step_dev != nullptr) step += *a.step_dev;
      }

      const int row_local = 32 * warp + lane;
      if (EPI == kWsPartial) {
        const int row = tile * kWsTileRows + row_local;
        float* dst = a.partials + static_cast<int64_t>(slice) * a.m * a.n + row;
#pragma unroll
        for (int t = 0; t < 64; ++t)
          if (t < a.m) dst[static_cast<int64_t>(t) * a.n] = v[t];
        if (a.peer_partials != nullptr) {   // the other GPU of the pair sums these slices too: store them there directly
          float* pdst = a.peer_partials + static_cast<int64_t>(slice) * a.m * a.n + row;
#pragma unroll
          for (int t = 0; t < 64; ++t)
            if (t < a.m) pdst[static_cast<int64_t>(t) * a.n] = v[t];
        }
      } else if (EPI == kWsBf16) {
        const int row = tile * kWsTileRows + row_local;
#pragma unroll
        for (int t = 0; t < 64; ++t)
          if (t < a.m) a.y[t * a.ldy + row] = __float2bfloat16_rn(v[t]);
      } else if (EPI == kWsSwiglu) {
        // rows 0..63 of the tile are gate rows, 64..127 the matching up rows: every thread parks its
        // row in shared memory, then all 128 threads share the SiLU*mul work (64 columns x 32 step rows
        // per pass, 16 outputs per thread)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          if (half * 32 >= a.m) break;
#pragma unroll
          for (int t = 0; t < 32; ++t) epi[row_local * 33 + t] = v[32 * half + t];
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const int c = threadIdx.x & 63;
          const int tg = threadIdx.x >> 6;          // 0 or 1: step rows [16*tg, 16*tg + 16)
          const int col = tile * 64 + c;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int tt = 16 * tg + i;
            const int r = 32 * half + tt;
            if (r < a.m) {
              const float gt = bf16_round(epi[c * 33 + tt]);
              const float up = bf16_round(epi[(64 + c) * 33 + tt]);
              const float s = gt * __frcp_rn(1.0f + __expf(-gt));
              a.y[r * a.ldy + col] = __float2bfloat16_rn(bf16_round(s) * up);
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      } else {
        // LM head: stage the tile, then each warp reduces 8-row groups of the step over the 128 vocabulary rows
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          if (half * 32 >= a.m) break;
#pragma unroll
          for (int t = 0; t < 32; ++t) epi[row_local * 33 + t] = v[32 * half + t];
          asm volatile("bar.sync 1, 128;" ::: "memory");
          for (int tt = warp; tt < 32 && 32 * half + tt < a.m; tt += 4) {
            const int r = 32 * half + tt;
            const float temp = a.temperatures[r / a.block];
            float mx = -INFINITY, bv = -INFINITY, bl = 0.f;
            int bi = 0x7fffffff;
            float lg[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int col = tile * kWsTileRows + lane + 32 * q;
              const float logit = bf16_round(epi[(lane + 32 * q) * 33 + tt]) / temp;
              lg[q] = logit;
              float noisy = logit;
              if (a.noise_mode == 1) noisy += a.noise[static_cast<int64_t>(r) * a.n + col];
              else if (a.noise_mode == 2) noisy += gumbel_noise(a.seed, step, r, col);
              mx = fmaxf(mx, logit);
              if (noisy > bv) { bv = noisy; bl = logit; bi = col; }   // ascending columns: first maximum kept
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
              a.part_f[static_cast<int64_t>(tile) * a.m + r] = make_float4(mx, se, bv, bl);
              a.part_i[static_cast<int64_t>(tile) * a.m + r] = bi;
              if (a.peer_part_f != nullptr) {
                a.peer_part_f[static_cast<int64_t>(tile) * a.m + r] = make_float4(mx, se, bv, bl);
                a.peer_part_i[static_cast<int64_t>(tile) * a.m + r] = bi;
              }
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      }
    }
  }

  if (threadIdx.x == 0) trace_event(EPI, 7);
  if (a.tp.peer_flags != nullptr && warp < 4) {
    // all four epilogue warps have issued their peer stores: publish them to the peer
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (threadIdx.x == 0) tp_signal(a.tp);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// ---- host side -----------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

struct MapKey {
  const void* ptr;
  int64_t rows, cols, ld;
  int box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h ^= static_cast<size_t>(k.rows) * 0x9e3779b97f4a7c15ull;
    h ^= static_cast<size_t>(k.cols) * 0xc2b2ae3d27d4eb4full;
    h ^= static_cast<size_t>(k.ld) * 0x165667b19e3779f9ull + static_cast<size_t>(k.box_rows);
    return h;
  }
};

// Tensor map of a row-major bf16 matrix [rows, cols] (row stride ld elements)
// read in boxes of box_rows x 64 columns with 128-byte swizzle.  Cached by
// (pointer, shape): weights and activation buffers live as long as the engine.
static bool get_tensor_map(const void* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{ptr, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return true;
  }
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return false;
  CUtensorMap m;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kWsBK), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  if (enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return true;
}

static int g_ws_sm_count = 0;

static int ws_smem_bytes(int stages, int ntok) {
  return 1024 + stages * (kWsWTileBytes + ntok * kWsBK * 2) + kWsEpiFloats * 4 + 16 * stages + 32 + 16;
}

// Shapes the tensor-core streaming kernel takes; anything else goes to the register-streaming kernel.
static bool ws_supported(int epi, int m, int n, int k, int64_t ldx) {
  if (m < 1 || m > (epi == kWsPartial ? kWsMaxRowsPartial : kWsMaxRows) || k % kWsBK != 0 || ldx % 8 != 0) return false;
  if (epi == kWsSwiglu) return (n / 2) % 64 == 0;
  return n % kWsTileRows == 0;
}

template <int EPI>
static int launch_ws(const bf16* x, int64_t ldx, const bf16* w, WsArgs& a, cudaStream_t st) {
  if (g_ws_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_ws_sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (g_ws_sm_count <= 0) g_ws_sm_count = 148;
  }
  a.ntok = (a.m + 15) / 16 * 16;
  a.chunks_total = a.k / kWsBK;
  a.chunks_per_slice = (a.chunks_total + a.ksplit - 1) / a.ksplit;
  a.tiles_n = (EPI == kWsSwiglu) ? a.inter / 64 : a.n / kWsTileRows;
  if (a.tiles_override > 0) a.tiles_n = a.tiles_override;
  const int budget = 227 * 1024;
  // Ring depth.  The LM head (one long stream) takes all the shared memory there is.  The projections of a layer
  // follow one another closely, and whatever a kernel requests before its dependency resolves competes with the
  // stream of the kernel it waits for: five stages for the slice form and six for the SiLU form measured best on
  // the 32-row step (1.726 -> 1.703 ms), although each kernel timed alone is 2 % slower or equal with them.
  int stages = 12;
  if (a.ntok <= 64) stages = EPI == kWsPartial ? 5 : (EPI == kWsSwiglu ? 6 : 12);
  while (stages > 2 && ws_smem_bytes(stages, a.ntok) > budget) --stages;
  if (stages > 16) stages = 16;
  a.stages = stages;
  const int smem = ws_smem_bytes(stages, a.ntok);

  CUtensorMap map_w, map_x;
  const int w_box_rows = (EPI == kWsSwiglu) ? 64 : kWsTileRows;
  if (!get_tensor_map(w, a.n, a.k, a.k, w_box_rows, &map_w)) return MDB_ERR_CUDA;
  if (!get_tensor_map(x, a.m, a.k, ldx, a.ntok, &map_x)) return MDB_ERR_CUDA;

  static PerDeviceOnce attr_once;
  const int dev = attr_once.slot();
  if (dev < 0) return MDB_ERR_CUDA;
  if (!attr_once.done[dev]) {
    if (cudaFuncSetAttribute(gemm_ws_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, budget) != cudaSuccess)
      return MDB_ERR_CUDA;
    attr_once.done[dev] = true;
  }
  const int tasks = a.tiles_n * a.ksplit;
  return mdb_launch(gemm_ws_kernel<EPI>, dim3(tasks < g_ws_sm_count ? tasks : g_ws_sm_count), dim3(kWsThreads), smem,
                    st, map_w, map_x, a);
}

}  // namespace mdb
