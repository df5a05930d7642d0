// y = x W^T for many rows (prefill, batched decode) on the 5th-generation tensor
// cores: persistent CTAs (one per SM), tiles of 128 step rows x 256 weight
// rows, tcgen05.mma M128 N256 K16 with the activation tile as A and the
// weight tile as B (both K-major, 128-byte swizzle, staged by TMA through a
// 4-stage ring of 48 KB), fp32 accumulators in tensor memory, double-buffered
// (2 x 256 columns = all 512) so the epilogue of a tile overlaps the main loop
// of the next.  Epilogue warps first (tcgen05.ld, one step row per thread),
// then the TMA producer warp and the MMA issue warp.  The bf16-store form has
// four epilogue warps; the SiLU and qkv forms eight (two per 32-lane quarter
// of tensor memory) and the LM-head form sixteen (four per quarter, 64
// columns each): their per-element work would otherwise outlast the main loop.
//
// Epilogues: bf16 store; SiLU(gate)*up for weight tiles made of 128 gate rows
// and their 128 up rows (the thread that owns a step row holds both halves);
// LM head + sampler: the thread that owns a step row turns its 256 logits of
// the vocabulary tile into one (max, sum-exp, best noisy value, its logit, its
// index) record, so logits never reach memory (nanovllm/layers/sampler.py:11-29
// on top of the LM head of nanovllm/models/sdar.py); qkv projection with the
// per-head q/k RMSNorm, rotary embedding and KV store (nanovllm/models/sdar.py:
// 73-82, nanovllm/layers/sdar_attention.py:37-38): a 256-column tile is two
// heads, and the thread that owns a step row holds a whole head of it.
// Tiles are ordered so that consecutive CTAs share a weight tile: it is read
// from HBM once and served from L2 to the others.
//
// PAIR form (taken from 2048 rows on): a cluster of two CTAs owns a tile of
// 256 step rows x 256 weight rows (tcgen05.mma.cta_group::2).  Each CTA stages
// its own 128 step rows (A) and its own 128 of the 256 weight rows (B) per k
// stage -- 32 KB instead of 48 KB for half the output -- and the MMA, issued by
// the leader CTA for both, reads the B halves of both CTAs, so shared-memory
// traffic per flop falls by a third; that traffic (operand reads + TMA fills
// above 128 B/clk at the tensor peak) is what bounds the one-CTA form.  Both
// producers' TMA loads complete on the leader's "full" barrier
// (cp.async.bulk.tensor with .cta_group::2), tcgen05.commit with a CTA mask
// arrives on the "empty" / "accumulator full" barriers of both CTAs, the
// peer's epilogue warps arrive on the leader's "accumulator empty" barrier
// through its cluster address, and a cluster barrier before the tensor memory
// is freed keeps either CTA's shared memory alive while the other may read it.
#include "mdb_common.cuh"

namespace mdb {

enum TcEpilogue { kTcBf16 = 0, kTcSwiglu = 1, kTcLmHead = 2, kTcQkvRope = 3 };

constexpr int kTcBM = 128, kTcBN = 256, kTcBK = 64;
constexpr int kTcStages = 4;
constexpr int kTcABytes = kTcBM * kTcBK * 2;   // 16 KB
constexpr int kTcBBytes = kTcBN * kTcBK * 2;   // 32 KB
constexpr int kTcPairStages = 6;               // PAIR: 16 KB of A + 16 KB of B per stage and CTA
constexpr int kTcLmEpiWarps = 16;
constexpr int kTcLmRecBytes = 2 * kTcLmEpiWarps * 32 * 5 * 4;    // two buffers of per-warp sampler records
__host__ __device__ constexpr int tc_epi_warps(int epi) { return epi == 2 ? kTcLmEpiWarps : 8; }
__host__ __device__ constexpr int tc_threads(int epi) { return (tc_epi_warps(epi) + 2) * 32; }

struct TcArgs {
  int m, n, k;        // n = output columns (swiglu: the intermediate size)
  int tiles_m, tiles_n;
  int inter;          // swiglu: first up row of the weight
  int n_fastest;      // tile order: 0 = consecutive CTAs share a weight tile, 1 = they share an activation tile
  bf16* y;
  int64_t ldy;
  // LM head + sampler
  const float* temperatures;   // per request
  int block;                   // step rows per request
  int noise_mode;              // 0 none, 2 counter-based Gumbel (explicit noise arrays take the materialising path)
  uint32_t seed, step;
  const uint32_t* step_dev;
  float4* part_f;              // [tiles_n][m] (max, sum exp, best noisy value, its logit)
  int* part_i;                 // [tiles_n][m] index of the best noisy value
  // qkv projection + q/k norm + rotary embedding + KV store
  int hq, hkv, max_pos;
  float eps;
  const int64_t* positions;
  const float* rope_table;     // [max_pos][64 cos | 64 sin]
  const bf16* q_norm_w;
  const bf16* k_norm_w;
  const int32_t* slot_mapping; // NULL: no cache write
  bf16* q_out;                 // [m][hq][128]
  bf16* k_out;                 // [m][hkv][128] or NULL
  bf16* v_out;
  bf16* k_cache;               // [slots][hkv][128]
  bf16* v_cache;
  int64_t num_slots;
  // tensor-parallel pair, bf16 epilogue: every output tile is also stored into the peer's memory (same
  // leading dimension), then the CTA raises its flag slot there (all null / zero on one GPU)
  bf16* y_peer;
  TpSignal tp;
  // LM head over a vocabulary shard (the weight pointer and n describe the shard): id of its first column, and
  // the peer's record arrays, which receive a copy of every record
  int col_base;
  float4* peer_part_f;
  int* peer_part_i;
  int grid;                    // CTAs launched (set by the launcher; the peer waits for that many flags)
  // bf16 form with few tiles: a cluster of ksplit CTAs shares one tile, each CTA a slice of k; the fp32 partial
  // tiles meet in shared memory (0 or 1: off)
  int ksplit;
};

constexpr int kTcParkStride = (kTcBN + 4) * 4;   // bytes per parked fp32 accumulator row: 16-byte pad against bank conflicts

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// warp-collective forms of the pair instructions
__device__ __forceinline__ void tma_load_2d_pair_w(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t leader_bar) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n\t}"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(leader_bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair_w(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "@q tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair_w(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t.reg .b16 m;\n\t"
      "mov.b16 m, 3;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}"
      ::"r"(bar)
      : "memory");
}

__device__ __forceinline__ float4 lds_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

template <int EPI, bool PAIR>
__global__ void __launch_bounds__(tc_threads(EPI), 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const TcArgs a) {
  extern __shared__ unsigned char tc_smem_raw[];
  constexpr int kStages = PAIR ? kTcPairStages : kTcStages;
  constexpr int kBBytes = PAIR ? kTcBBytes / 2 : kTcBBytes;      // PAIR: this CTA's 128 of the tile's 256 weight rows
  constexpr int kRowsPerTile = PAIR ? 2 * kTcBM : kTcBM;
  const uint32_t raw = smem_u32(tc_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;                  // PAIR: same offset in both CTAs (same kernel, same layout)
  unsigned char* gen_base = tc_smem_raw + (base - raw);
  const uint32_t a_tiles = base;
  const uint32_t b_tiles = base + kStages * kTcABytes;
  const uint32_t bars_off = kStages * (kTcABytes + kBBytes);
  const uint32_t bars = base + bars_off;
  const uint32_t bar_full = bars, bar_empty = bars + 8 * kStages;
  const uint32_t bar_acc_full = bars + 16 * kStages, bar_acc_empty = bar_acc_full + 16;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(gen_base + bars_off + 16 * kStages + 32);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kEpiWarps = tc_epi_warps(EPI);
  constexpr int kProducerWarp = kEpiWarps, kMmaWarp = kEpiWarps + 1;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;           // 0 = the CTA that issues the MMAs
  // split-k clusters (bf16 form, single-CTA tiles): ks CTAs per tile, this one takes k chunks [c_begin, c_end)
  const int ks = (EPI == kTcBf16 && !PAIR && a.ksplit > 1) ? a.ksplit : 1;
  const uint32_t kr = ks > 1 ? cluster_ctarank() : 0u;
  const int work0 = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x) / ks;
  const int work_stride = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x) / ks;
  const int tiles = a.tiles_m * a.tiles_n;
  const int kchunks = a.k / kTcBK;
  const int c_begin = static_cast<int>(kr) * kchunks / ks, c_end = (static_cast<int>(kr) + 1) * kchunks / ks;
  int parked_tile = -1;                                          // split-k: the tile whose partial this CTA parked

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);      // PAIR: used in the leader; its producer's arrive + bytes from both CTAs
      mbar_init(bar_empty + 8 * s, 1);     // PAIR: one commit, multicast to both CTAs
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, PAIR ? 2 * kEpiWarps : kEpiWarps);   // PAIR: the epilogue warps of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    const uint32_t slot = smem_u32(const_cast<uint32_t*>(&misc[0]));
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(512u) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(512u) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  if (PAIR) cluster_sync_all();            // the barriers of both CTAs exist before anyone signals across
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = misc[0];
  // where an epilogue warp reports that it has drained an accumulator buffer
  const uint32_t acc_empty_target = PAIR ? map_to_cta(bar_acc_empty, 0) : bar_acc_empty;
  auto arrive_acc_empty = [&](int acc_buf) {
    if (PAIR) mbar_arrive_cluster(acc_empty_target + 8 * acc_buf);
    else mbar_arrive(acc_empty_target + 8 * acc_buf);
  };

  if (warp == kProducerWarp) {
    // the whole warp walks the loop (warp-uniform operands), one elected lane issues each instruction
    const uint32_t full_target = PAIR ? map_to_cta(bar_full, 0) : bar_full;
    auto tile_of = [&](int t, int& tn, int& tm) {
      tn = a.n_fastest ? t % a.tiles_n : t / a.tiles_m;   // consecutive CTAs share a weight tile, or,
      tm = a.n_fastest ? t / a.tiles_n : t % a.tiles_m;   // when the activations outgrow L2, an activation tile
    };
    // a stage's barrier expects the bytes of both operands; the weight tile may be requested long before the
    // activation tile
    auto load_weights = [&](int stage, int c, int tn) {
      const uint32_t full = full_target + 8 * stage;
      const uint32_t bdst = b_tiles + stage * kBBytes;
      if (PAIR) {
        // own 128 weight rows (SiLU form: the leader holds the gate rows, the peer the up rows)
        if (rank == 0) mbar_arrive_expect_tx_w(bar_full + 8 * stage, 2 * (kTcABytes + kBBytes));
        const int brow = EPI == kTcSwiglu ? (rank == 0 ? tn * 128 : a.inter + tn * 128)
                                          : tn * kTcBN + static_cast<int>(rank) * 128;
        tma_load_2d_pair_w(bdst, &map_w, c * kTcBK, brow, full);
      } else {
        mbar_arrive_expect_tx_w(full, kTcABytes + kTcBBytes);
        if (EPI == kTcSwiglu) {
          tma_load_2d_w(bdst, &map_w, c * kTcBK, tn * 128, full);                             // 128 gate rows
          tma_load_2d_w(bdst + kTcBBytes / 2, &map_w, c * kTcBK, a.inter + tn * 128, full);   // their up rows
        } else {
          tma_load_2d_w(bdst, &map_w, c * kTcBK, tn * kTcBN, full);
        }
      }
    };
    auto load_rows = [&](int stage, int c, int tm) {
      const uint32_t full = full_target + 8 * stage;
      const uint32_t adst = a_tiles + stage * kTcABytes;
      if (PAIR) tma_load_2d_pair_w(adst, &map_x, c * kTcBK, tm * kRowsPerTile + static_cast<int>(rank) * kTcBM, full);
      else tma_load_2d_w(adst, &map_x, c * kTcBK, tm * kTcBM, full);
    };
    // Weights are written by no kernel of a step: the first ring-full of weight tiles is requested before the
    // dependency wait (the stages are fresh, nothing to wait for), the activation tiles follow after it.
    int early = 0;
    if (work0 < tiles) {
      int tn, tm;
      tile_of(work0, tn, tm);
      early = c_end - c_begin < kStages ? c_end - c_begin : kStages;
      for (int c = 0; c < early; ++c) load_weights(c, c_begin + c, tn);
    }
    pdl_wait();   // activations come from the preceding kernel
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int t = work0; t < tiles && ok; t += work_stride) {
      int tn, tm;
      tile_of(t, tn, tm);
      for (int c = c_begin; c < c_end; ++c) {
        if (early > 0) {
          --early;                       // weight tile of this stage already on its way
        } else {
          if (!mbar_wait_w(bar_empty + 8 * stage, phase ^ 1)) { ok = false; break; }
          load_weights(stage, c, tn);
        }
        load_rows(stage, c, tm);
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
    if (!ok && lane == 0) report_status(MDB_STATUS_WAIT_TIMEOUT);
  } else if (warp == kMmaWarp) {
    if (rank == 0) {
      // bf16 x bf16 -> fp32, K-major operands, M = 128 (PAIR: 256, 128 per CTA), N = 256
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kTcBN >> 3) << 17) |
                             (static_cast<uint32_t>(kRowsPerTile >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = work0; t < tiles && ok; t += work_stride) {
        if (!mbar_wait_w(bar_acc_empty + 8 * acc, acc_phase ^ 1)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kTcBN;
        for (int c = c_begin; c < c_end; ++c) {
          if (!mbar_wait_w(bar_full + 8 * stage, phase)) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = umma_desc_sw128(a_tiles + stage * kTcABytes);
          const uint64_t bdesc = umma_desc_sw128(b_tiles + stage * kBBytes);
#pragma unroll
          for (int k16 = 0; k16 < kTcBK / 16; ++k16) {
            if (PAIR) umma_bf16_pair_w(d_tmem, adesc + 2 * k16, bdesc + 2 * k16, idesc, (c > c_begin || k16 > 0) ? 1u : 0u);
            else umma_bf16_w(d_tmem, adesc + 2 * k16, bdesc + 2 * k16, idesc, (c > c_begin || k16 > 0) ? 1u : 0u);
          }
          if (PAIR) umma_commit_pair_w(bar_empty + 8 * stage);
          else umma_commit_w(bar_empty + 8 * stage);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (PAIR) umma_commit_pair_w(bar_acc_full + 8 * acc);
        else umma_commit_w(bar_acc_full + 8 * acc);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok && lane == 0) report_status(MDB_STATUS_WAIT_TIMEOUT);
    }
  } else {
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t acc_phase_tile = 0;   // tiles done (LM head: picks the record buffer)
    pdl_wait();   // the output buffer may still be read by the preceding kernel
    for (int t = work0; t < tiles; t += work_stride) {
      const int tn = a.n_fastest ? t % a.tiles_n : t / a.tiles_m;
      const int tm = a.n_fastest ? t / a.tiles_n : t % a.tiles_m;
      // q/k-norm + rotation form: this lane's position (-1: none, or outside the table) and the request for the
      // first quarter of the warp's cos | sin rows go out before the accumulator is waited for
      const uint32_t rope_smem = base + bars_off + 256 + warp * 4096;
      int rope_pos = -1;
      auto rope_fill = [&](int p) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = 4 * i + (lane >> 3);
          const int j = lane & 7;                       // 16-byte piece of the row's pass: 0..3 cos, 4..7 sin
          const int pr = __shfl_sync(0xffffffffu, rope_pos, r);
          if (pr >= 0) {
            const float* src = a.rope_table + static_cast<int64_t>(pr) * kHeadDim + (j >> 2) * 64 + 16 * p + 4 * (j & 3);
            const uint32_t dst = rope_smem + r * 128 + ((static_cast<uint32_t>(j) ^ (r & 7u)) << 4);
            asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
          }
        }
      };
      if (EPI == kTcQkvRope) {
        const int prow = tm * kRowsPerTile + static_cast<int>(rank) * kTcBM + 32 * (warp & 3) + lane;
        const int phead = 2 * tn + (warp >> 2);
        if (phead < a.hq + a.hkv) {
          if (prow < a.m) {
            const int64_t pos = a.positions[prow];
            rope_pos = (pos >= 0 && pos < a.max_pos) ? static_cast<int>(pos) : -1;
          }
          rope_fill(0);
        }
      }
      bool ok = mbar_wait(bar_acc_full + 8 * acc, acc_phase);
      ok = __all_sync(0xffffffffu, ok);
      // LM head: the warps of a quarter meet at a named barrier below, so they must agree on giving up
      if (EPI == kTcLmHead) ok = named_bar_and(5 + (warp & 3), 128, ok);
      if (!ok) {
        if (EPI == kTcQkvRope) asm volatile("cp.async.wait_all;" ::: "memory");
        if (lane == 0) report_status(MDB_STATUS_WAIT_TIMEOUT);
        break;
      }
      tc_fence_after();
      const int quarter = warp & 3;       // the 32 tensor-memory lanes this warp may read
      const uint32_t taddr = tmem_base + acc * kTcBN + (static_cast<uint32_t>(32 * quarter) << 16);
      const int row = tm * kRowsPerTile + static_cast<int>(rank) * kTcBM + 32 * quarter + lane;
      if (EPI == kTcBf16 && ks > 1) {
        // split-k cluster: every MMA of this CTA has completed, so the operand ring is idle (a cluster owns one
        // tile, nothing more will be loaded): park the fp32 partial tile there, one row per thread
        const uint32_t park = a_tiles + (32 * quarter + lane) * kTcParkStride + (warp >> 2) * (kTcBN / 2) * 4;
#pragma unroll 1
        for (int c = 0; c < kTcBN / 64; ++c) {
          float v0[16], v1[16];
          tmem_ld16(taddr + (warp >> 2) * (kTcBN / 2) + 32 * c, v0);
          tmem_ld16(taddr + (warp >> 2) * (kTcBN / 2) + 32 * c + 16, v1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(park + (32 * c + 4 * i) * 4), "f"(v0[4 * i]),
                         "f"(v0[4 * i + 1]), "f"(v0[4 * i + 2]), "f"(v0[4 * i + 3])
                         : "memory");
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(park + (32 * c + 16 + 4 * i) * 4), "f"(v1[4 * i]),
                         "f"(v1[4 * i + 1]), "f"(v1[4 * i + 2]), "f"(v1[4 * i + 3])
                         : "memory");
          }
        }
        parked_tile = t;
        break;
      }
      if (EPI == kTcBf16) {
        bf16* dst = a.y + static_cast<int64_t>(row) * a.ldy + tn * kTcBN;
        // Tensor-parallel pair: the copy for the peer is staged in shared memory, 32 rows x 64 columns per warp,
        // and leaves as 128-byte row segments (four rows per store instruction): over NVLink the 16-byte pieces
        // a thread holds of its own row would travel one by one.
        const bool peer_staged = a.y_peer != nullptr && (tn + 1) * kTcBN <= a.n;
        const uint32_t stage_smem = base + bars_off + 256 + warp * 4096;
        // two warps per quarter of tensor memory, 128 of the tile's 256 columns each
        const int c0 = (warp >> 2) * (kTcBN / 64);
#pragma unroll 1
        for (int c = c0; c < c0 + kTcBN / 64; ++c) {
          float v0[16], v1[16];
          tmem_ld16(taddr + 32 * c, v0);
          tmem_ld16(taddr + 32 * c + 16, v1);
          tmem_ld_wait();
          const int col = tn * kTcBN + 32 * c;
          if (row < a.m) {
            if (col + 32 <= a.n) {
              uint4 o[4];
              o[0] = make_uint4(pack_bf16x2(v0[0], v0[1]), pack_bf16x2(v0[2], v0[3]), pack_bf16x2(v0[4], v0[5]), pack_bf16x2(v0[6], v0[7]));
              o[1] = make_uint4(pack_bf16x2(v0[8], v0[9]), pack_bf16x2(v0[10], v0[11]), pack_bf16x2(v0[12], v0[13]), pack_bf16x2(v0[14], v0[15]));
              o[2] = make_uint4(pack_bf16x2(v1[0], v1[1]), pack_bf16x2(v1[2], v1[3]), pack_bf16x2(v1[4], v1[5]), pack_bf16x2(v1[6], v1[7]));
              o[3] = make_uint4(pack_bf16x2(v1[8], v1[9]), pack_bf16x2(v1[10], v1[11]), pack_bf16x2(v1[12], v1[13]), pack_bf16x2(v1[14], v1[15]));
              uint4* d4 = reinterpret_cast<uint4*>(dst + 32 * c);
              d4[0] = o[0]; d4[1] = o[1]; d4[2] = o[2]; d4[3] = o[3];
              if (a.y_peer != nullptr && !peer_staged) {   // ragged right edge: the same 64 bytes straight to the peer
                uint4* p4 = reinterpret_cast<uint4*>(a.y_peer + static_cast<int64_t>(row) * a.ldy + tn * kTcBN + 32 * c);
                p4[0] = o[0]; p4[1] = o[1]; p4[2] = o[2]; p4[3] = o[3];
              }
              if (peer_staged) {
                // 16-byte piece s of a staged row sits at piece s ^ (row & 7): no bank conflicts either way
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const uint32_t piece = static_cast<uint32_t>(4 * (c & 1) + i) ^ static_cast<uint32_t>(lane & 7);
                  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage_smem + lane * 128 + (piece << 4)),
                               "r"(o[i].x), "r"(o[i].y), "r"(o[i].z), "r"(o[i].w)
                               : "memory");
                }
              }
            } else {
              bf16* pdst = a.y_peer != nullptr ? a.y_peer + static_cast<int64_t>(row) * a.ldy + tn * kTcBN : nullptr;
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                if (col + i < a.n) {
                  dst[32 * c + i] = __float2bfloat16_rn(v0[i]);
                  if (pdst != nullptr) pdst[32 * c + i] = __float2bfloat16_rn(v0[i]);
                }
                if (col + 16 + i < a.n) {
                  dst[32 * c + 16 + i] = __float2bfloat16_rn(v1[i]);
                  if (pdst != nullptr) pdst[32 * c + 16 + i] = __float2bfloat16_rn(v1[i]);
                }
              }
            }
          }
          if (peer_staged && (c & 1)) {
            __syncwarp();
            const int row0 = tm * kRowsPerTile + static_cast<int>(rank) * kTcBM + 32 * quarter;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int r = 4 * it + (lane >> 3);
              const uint32_t piece = static_cast<uint32_t>(lane & 7) ^ static_cast<uint32_t>(r & 7);
              uint4 o;
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(o.x), "=r"(o.y), "=r"(o.z), "=r"(o.w)
                           : "r"(stage_smem + r * 128 + (piece << 4)));
              if (row0 + r < a.m)
                *reinterpret_cast<uint4*>(a.y_peer + static_cast<int64_t>(row0 + r) * a.ldy + tn * kTcBN + 32 * (c - 1) +
                                          8 * (lane & 7)) = o;
            }
            __syncwarp();
          }
        }
      } else if (EPI == kTcSwiglu) {
        // columns [0,128) gate, [128,256) up of the same 128 intermediate columns; two warps per quarter,
        // 64 of the 128 outputs each (with four warps the SiLU work outlasts the main loop)
        const int grp = warp >> 2;
        bf16* dst = a.y + static_cast<int64_t>(row) * a.ldy + tn * 128 + 64 * grp;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          float g[16], u[16];
          tmem_ld16(taddr + 64 * grp + 16 * c, g);
          tmem_ld16(taddr + 128 + 64 * grp + 16 * c, u);
          tmem_ld_wait();
          if (row < a.m) {
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float r[2];
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const float gt = bf16_round(g[2 * i + e]);
                const float up = bf16_round(u[2 * i + e]);
                const float sl = gt * rcp_approx(1.0f + __expf(-gt));   // fp32 SiLU, rounded to bf16 below
                r[e] = bf16_round(sl) * up;
              }
              o[i] = pack_bf16x2(r[0], r[1]);
            }
            uint4* d4 = reinterpret_cast<uint4*>(dst + 16 * c);
            d4[0] = make_uint4(o[0], o[1], o[2], o[3]);
            d4[1] = make_uint4(o[4], o[5], o[6], o[7]);
          }
        }
      }
      if (EPI == kTcQkvRope) {
        // this warp: head 2 tn + g of the fused q|k|v output for its 32 step rows.  Everything the projection,
        // the norm and the rotation leave is bf16, so a row's head lives packed in 64 registers throughout.
        const int grp = warp >> 2;
        const int head = 2 * tn + grp;
        const int nheads = a.hq + 2 * a.hkv;
        const bool is_q = head < a.hq;
        const bool is_k = !is_q && head < a.hq + a.hkv;
        const bool live = row < a.m && head < nheads;
        uint32_t pk[kHeadDim / 2];
        float ss0 = 0.f, ss1 = 0.f, ss2 = 0.f, ss3 = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float t0[16], t1[16];
          tmem_ld16(taddr + kHeadDim * grp + 32 * c, t0);
          tmem_ld16(taddr + kHeadDim * grp + 32 * c + 16, t1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            // the projection's bf16 output; sum of squares over the rounded values in four interleaved chains
            pk[16 * c + i / 2] = pack_bf16x2(t0[i], t0[i + 1]);
            pk[16 * c + i / 2 + 1] = pack_bf16x2(t0[i + 2], t0[i + 3]);
            const float2 f0 = unpack_bf16x2(pk[16 * c + i / 2]), f1 = unpack_bf16x2(pk[16 * c + i / 2 + 1]);
            ss0 = fmaf(f0.x, f0.x, ss0); ss1 = fmaf(f0.y, f0.y, ss1);
            ss2 = fmaf(f1.x, f1.x, ss2); ss3 = fmaf(f1.y, f1.y, ss3);
          }
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            pk[16 * c + 8 + i / 2] = pack_bf16x2(t1[i], t1[i + 1]);
            pk[16 * c + 8 + i / 2 + 1] = pack_bf16x2(t1[i + 2], t1[i + 3]);
            const float2 f0 = unpack_bf16x2(pk[16 * c + 8 + i / 2]), f1 = unpack_bf16x2(pk[16 * c + 8 + i / 2 + 1]);
            ss0 = fmaf(f0.x, f0.x, ss0); ss1 = fmaf(f0.y, f0.y, ss1);
            ss2 = fmaf(f1.x, f1.x, ss2); ss3 = fmaf(f1.y, f1.y, ss3);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) arrive_acc_empty(acc);
        if (is_q || is_k) {          // warp-uniform: a warp owns one head
          if (live) {
            const float rstd = 1.0f / sqrtf(((ss0 + ss1) + (ss2 + ss3)) / static_cast<float>(kHeadDim) + a.eps);
            const uint4* nw = reinterpret_cast<const uint4*>(is_q ? a.q_norm_w : a.k_norm_w);
#pragma unroll
            for (int c = 0; c < kHeadDim / 8; ++c) {
              const uint4 w8 = __ldg(nw + c);
              const uint32_t ws[4] = {w8.x, w8.y, w8.z, w8.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = unpack_bf16x2(pk[4 * c + j]), wf = unpack_bf16x2(ws[j]);
                pk[4 * c + j] = pack_bf16x2(bf16_round(f.x * rstd) * wf.x, bf16_round(f.y * rstd) * wf.y);
              }
            }
          }
          // Rotation: the cos | sin rows of the warp's 32 positions come through this warp's 4 KB of shared
          // memory in four passes of 16 channel pairs, fetched as 64-byte segments (eight lanes per row) and read
          // back one row per lane; 16-byte piece j of row r sits at piece j ^ (r & 7), conflict-free both ways.
          // Pass 0 was requested before the accumulator wait.
          const bool pos_bad = live && rope_pos < 0;
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            asm volatile("cp.async.wait_all;" ::: "memory");
            __syncwarp();
            float4 co[4], si[4];
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              co[c4] = lds_f4(rope_smem + lane * 128 + ((static_cast<uint32_t>(c4) ^ (lane & 7u)) << 4));
              si[c4] = lds_f4(rope_smem + lane * 128 + ((static_cast<uint32_t>(4 + c4) ^ (lane & 7u)) << 4));
            }
            __syncwarp();
            if (p < 3) rope_fill(p + 1);
            if (live && !pos_bad) {
#pragma unroll
              for (int c4 = 0; c4 < 4; ++c4) {
                const int c = 4 * p + c4;
                const float cc[4] = {co[c4].x, co[c4].y, co[c4].z, co[c4].w};
                const float sn[4] = {si[c4].x, si[c4].y, si[c4].z, si[c4].w};
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) {
                  const float2 lo = unpack_bf16x2(pk[2 * c + h2]), hi = unpack_bf16x2(pk[32 + 2 * c + h2]);
                  // products rounded separately, as un-fused fp32 tensor ops do
                  const float lx = __fsub_rn(__fmul_rn(lo.x, cc[2 * h2]), __fmul_rn(hi.x, sn[2 * h2]));
                  const float ly = __fsub_rn(__fmul_rn(lo.y, cc[2 * h2 + 1]), __fmul_rn(hi.y, sn[2 * h2 + 1]));
                  const float hx = __fadd_rn(__fmul_rn(hi.x, cc[2 * h2]), __fmul_rn(lo.x, sn[2 * h2]));
                  const float hy = __fadd_rn(__fmul_rn(hi.y, cc[2 * h2 + 1]), __fmul_rn(lo.y, sn[2 * h2 + 1]));
                  pk[2 * c + h2] = pack_bf16x2(lx, ly);
                  pk[32 + 2 * c + h2] = pack_bf16x2(hx, hy);
                }
              }
            }
          }
          if (pos_bad) report_status(MDB_STATUS_BAD_POSITION);
        }
        // Stores: a thread holds a whole head of its own row, which would leave as 16-byte pieces of 32 different
        // rows per instruction.  The warp turns its 32 x 128 elements around in its 4 KB of shared memory, half a
        // head at a time, and writes 128-byte row segments, four rows per instruction.
        if (head < nheads) {         // warp-uniform
          const int row0 = row - lane;
          const int kvh = is_k ? head - a.hq : head - a.hq - a.hkv;
          bf16* contiguous = is_q ? a.q_out : (is_k ? a.k_out : a.v_out);
          const int heads_out = is_q ? a.hq : a.hkv;
          const int head_out = is_q ? head : kvh;
          bf16* cache = is_q ? nullptr : (is_k ? a.k_cache : a.v_cache);
          int my_slot = -1;
          if (!is_q && a.slot_mapping != nullptr && live) {
            const int slot = a.slot_mapping[row];
            if (slot >= 0 && slot < a.num_slots) my_slot = slot;
            else if (slot != -1) report_status(MDB_STATUS_BAD_SLOT);
          }
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rope_smem + lane * 128 +
                                                                            ((static_cast<uint32_t>(j) ^ (lane & 7u)) << 4)),
                           "r"(pk[32 * hf + 4 * j]), "r"(pk[32 * hf + 4 * j + 1]), "r"(pk[32 * hf + 4 * j + 2]),
                           "r"(pk[32 * hf + 4 * j + 3])
                           : "memory");
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = 4 * i + (lane >> 3);
              const int j = lane & 7;
              uint4 o;
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(o.x), "=r"(o.y), "=r"(o.z), "=r"(o.w)
                           : "r"(rope_smem + r * 128 + ((static_cast<uint32_t>(j) ^ (r & 7u)) << 4)));
              const int slot_r = __shfl_sync(0xffffffffu, my_slot, r);
              const int rr = row0 + r;
              if (rr < a.m) {
                const int col = 64 * hf + 8 * j;
                if (contiguous != nullptr)
                  *reinterpret_cast<uint4*>(contiguous + (static_cast<int64_t>(rr) * heads_out + head_out) * kHeadDim + col) = o;
                if (slot_r >= 0)
                  *reinterpret_cast<uint4*>(cache + (static_cast<int64_t>(slot_r) * a.hkv + kvh) * kHeadDim + col) = o;
              }
            }
            __syncwarp();
          }
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        continue;
      }
      if (EPI == kTcLmHead) {
        // this warp: columns [64 g, 64 g + 64) of the tile for its 32 step rows
        const int grp = warp >> 2;
        const bool live = row < a.m;
        const float inv_temp = __frcp_rn(a.temperatures[(live ? row : 0) / a.block]);
        const uint32_t step = a.step + (a.step_dev != nullptr ? *a.step_dev : 0u);
        const uint32_t key = gumbel_row_key(a.seed, step, row);
        constexpr float kLog2e = 1.4426950408889634f;
        float mx = -INFINITY, se = 0.f, bv = -INFINITY, bl = 0.f;
        int bi = 0x7fffffff;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          const int col0 = tn * kTcBN + 64 * grp + 32 * half;
          if (col0 >= a.n) break;            // uniform; the last vocabulary tile may be partly outside
          float v[32];
          tmem_ld16(taddr + 64 * grp + 32 * half, *reinterpret_cast<float(*)[16]>(v));
          tmem_ld16(taddr + 64 * grp + 32 * half + 16, *reinterpret_cast<float(*)[16]>(v + 16));
          tmem_ld_wait();
          const bool full = col0 + 32 <= a.n;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            v[i] = bf16_round(v[i]) * inv_temp;
            if (!full && col0 + i >= a.n) v[i] = -INFINITY;
          }
          float m0 = fmaxf(v[0], v[1]), m1 = fmaxf(v[2], v[3]);
#pragma unroll
          for (int i = 4; i < 32; i += 4) {
            m0 = fmaxf(m0, fmaxf(v[i], v[i + 1]));
            m1 = fmaxf(m1, fmaxf(v[i + 2], v[i + 3]));
          }
          const float nm = fmaxf(mx, fmaxf(m0, m1));
          const float nm2 = nm * kLog2e;
          float s0 = 0.f, s1 = 0.f;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            s0 += ex2_approx(fmaf(v[i], kLog2e, -nm2));          // 2^-inf = 0 for columns outside
            s1 += ex2_approx(fmaf(v[i + 1], kLog2e, -nm2));
          }
          se = (mx == -INFINITY ? 0.f : se * ex2_approx(fmaf(mx, kLog2e, -nm2))) + s0 + s1;
          mx = nm;
          if (a.noise_mode == 2) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float noisy = v[i] + gumbel_from_key(key, a.col_base + col0 + i);   // -inf stays -inf
              if (noisy > bv) { bv = noisy; bl = v[i]; bi = a.col_base + col0 + i; }    // ascending columns: first maximum kept
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (v[i] > bv) { bv = v[i]; bl = v[i]; bi = a.col_base + col0 + i; }
          }
        }
        // the four warps of a quarter merge their records through shared memory (two buffers, one barrier per tile)
        float* rec = reinterpret_cast<float*>(gen_base + bars_off + 256) + ((acc_phase_tile & 1) * kTcLmEpiWarps + warp) * 160;
        rec[lane] = mx; rec[32 + lane] = se; rec[64 + lane] = bv; rec[96 + lane] = bl;
        rec[128 + lane] = __int_as_float(bi);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) arrive_acc_empty(acc);
        asm volatile("bar.sync %0, 128;" ::"r"(1 + quarter) : "memory");
        if (grp == 0) {
          SampleRec r = {mx, se, bv, bl, bi};
#pragma unroll
          for (int g2 = 1; g2 < 4; ++g2) {
            const float* o = rec + g2 * 4 * 160;
            const SampleRec t = {o[lane], o[32 + lane], o[64 + lane], o[96 + lane], __float_as_int(o[128 + lane])};
            merge_rec(r, t);
          }
          if (live) {
            a.part_f[static_cast<int64_t>(tn) * a.m + row] = make_float4(r.mx, r.se, r.bv, r.bl);
            a.part_i[static_cast<int64_t>(tn) * a.m + row] = r.bi;
            if (a.peer_part_f != nullptr) {      // consecutive rows: 512 bytes per warp over NVLink
              a.peer_part_f[static_cast<int64_t>(tn) * a.m + row] = make_float4(r.mx, r.se, r.bv, r.bl);
              a.peer_part_i[static_cast<int64_t>(tn) * a.m + row] = r.bi;
            }
          }
        }
        ++acc_phase_tile;
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        continue;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) arrive_acc_empty(acc);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  if (EPI == kTcBf16 && ks > 1) {
    // every CTA of the cluster has parked its partial tile; CTA kr sums rows [kr, kr + 1) * 128 / ks of all of
    // them in CTA order (so the result does not depend on timing), rounds to bf16 and stores row segments
    tc_fence_before();
    cluster_sync_all();
    if (warp < kEpiWarps) {
      parked_tile = __shfl_sync(0xffffffffu, parked_tile, 0);
      if (parked_tile >= 0) {
        const int tn = a.n_fastest ? parked_tile % a.tiles_n : parked_tile / a.tiles_m;
        const int tm = a.n_fastest ? parked_tile / a.tiles_n : parked_tile % a.tiles_m;
        const int rows_per = kTcBM / ks;
        const int r0 = static_cast<int>(kr) * rows_per;
        for (int item = threadIdx.x; item < rows_per * (kTcBN / 4); item += kEpiWarps * 32) {
          const int r = r0 + item / (kTcBN / 4), c4 = item % (kTcBN / 4);
          // all remote loads of an element go out together (a remote read is several hundred cycles), the sum
          // then runs in CTA order
          float4 v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (j < ks)
              asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                           : "=f"(v[j].x), "=f"(v[j].y), "=f"(v[j].z), "=f"(v[j].w)
                           : "r"(map_to_cta(a_tiles + r * kTcParkStride + c4 * 16, static_cast<uint32_t>(j))));
          }
          float4 sum = v[0];
#pragma unroll
          for (int j = 1; j < 8; ++j)
            if (j < ks) { sum.x += v[j].x; sum.y += v[j].y; sum.z += v[j].z; sum.w += v[j].w; }
          const int grow = tm * kTcBM + r, col = tn * kTcBN + 4 * c4;
          if (grow < a.m) {
            bf16* dst = a.y + static_cast<int64_t>(grow) * a.ldy + col;
            if (col + 4 <= a.n) {
              *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(sum.x, sum.y), pack_bf16x2(sum.z, sum.w));
            } else {
              const float e[4] = {sum.x, sum.y, sum.z, sum.w};
              for (int i = 0; i < 4; ++i)
                if (col + i < a.n) dst[i] = __float2bfloat16_rn(e[i]);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  if (PAIR || ks > 1) cluster_sync_all();  // no CTA leaves while another may still read its shared memory
  else __syncthreads();
  if ((EPI == kTcBf16 || EPI == kTcLmHead) && threadIdx.x == 0) tp_signal(a.tp);   // all peer stores of this CTA were issued before the barrier
  if (warp == kMmaWarp) {
    tc_fence_after();
    if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// Shapes this kernel takes: k a multiple of 64, 16-byte aligned rows; swiglu additionally inter % 128 == 0.
static bool tc_supported(int epi, int m, int n, int k, int64_t ldx, int64_t ldy) {
  if (m < 1 || k % kTcBK != 0 || ldx % 8 != 0) return false;
  if (epi == kTcLmHead) return true;
  if (epi == kTcQkvRope) return n % kHeadDim == 0;
  if (ldy % 8 != 0) return false;
  if (epi == kTcSwiglu) return n % 128 == 0;
  return n % 8 == 0;
}

template <int EPI, bool PAIR>
static int launch_tc_impl(const bf16* x, int64_t ldx, const bf16* w, int w_rows, TcArgs& a, cudaStream_t st) {
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  constexpr int kRowsPerTile = PAIR ? 2 * kTcBM : kTcBM;
  // after the barriers: sampler records (LM head), or 4 KB per epilogue warp: the peer's staged tile (bf16 form),
  // the cos | sin rows and the turned-around stores (q/k-norm + rotation form)
  constexpr int kTail = (EPI == kTcQkvRope || EPI == kTcBf16) ? tc_epi_warps(EPI) * 4096 : kTcLmRecBytes;
  constexpr int kSmem = 1024 + (PAIR ? kTcPairStages * (kTcABytes + kTcBBytes / 2) : kTcStages * (kTcABytes + kTcBBytes)) +
                        256 + kTail;
  static_assert(kSmem <= 232448, "shared memory of the tile GEMM");
  a.tiles_m = (a.m + kRowsPerTile - 1) / kRowsPerTile;
  a.tiles_n = (EPI == kTcSwiglu) ? a.n / 128 : (a.n + kTcBN - 1) / kTcBN;
  // Activations that do not fit in L2 next to the weights (a 16K-row step of down_proj: 201 MB) would be
  // re-read from HBM once per weight tile; then the tiles of one activation band run back to back instead.
  a.n_fastest = static_cast<int64_t>(a.m) * a.k * 2 > (96ll << 20) &&
                static_cast<int64_t>(w_rows) * a.k * 2 < static_cast<int64_t>(a.m) * a.k * 2 ? 1 : 0;
  CUtensorMap map_x, map_w;
  if (!get_tensor_map(x, a.m, a.k, ldx, kTcBM, &map_x)) return MDB_ERR_CUDA;
  if (!get_tensor_map(w, w_rows, a.k, a.k, (PAIR || EPI == kTcSwiglu) ? 128 : kTcBN, &map_w)) return MDB_ERR_CUDA;
  static PerDeviceOnce attr_once;
  const int dev = attr_once.slot();
  if (dev < 0) return MDB_ERR_CUDA;
  if (!attr_once.done[dev]) {
    if (cudaFuncSetAttribute(gemm_tc_kernel<EPI, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess)
      return MDB_ERR_CUDA;
    attr_once.done[dev] = true;
  }
  const int tiles = a.tiles_m * a.tiles_n;
  a.grid = tiles < sm_count ? tiles : sm_count;
  a.ksplit = 1;
  if (!PAIR && EPI == kTcBf16 && a.y_peer == nullptr && a.tp.peer_flags == nullptr) {
    // Few tiles (a projection onto 2048 columns has 8 per 128 step rows): clusters of 2, 4 or 8 CTAs split k so
    // that about every SM streams a share of the weight; at least eight 64-wide chunks per slice.
    // A cluster lives inside one processing cluster of the GPU, so fewer clusters of 8 fit than SMs / 8: a split is
    // only taken when all its clusters are resident at once (a second wave would double the time).
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(tc_threads(EPI));
    cfg.dynamicSmemBytes = kSmem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static int max_clusters[4] = {0, 0, 0, 0};     // resident clusters of 2, 4, 8 CTAs (index = log2)
    int ksplit = 8, lg = 3;
    for (; ksplit > 1; ksplit >>= 1, --lg) {
      if (a.k / kTcBK < 8 * ksplit) continue;
      if (max_clusters[lg] == 0) {
        int n = 0;
        cfg.gridDim = dim3(sm_count / ksplit * ksplit);
        attr[0].val.clusterDim.x = ksplit;
        cfg.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_kernel<EPI, PAIR>, &cfg) != cudaSuccess || n <= 0) n = -1;
        max_clusters[lg] = n;
      }
      if (tiles <= max_clusters[lg]) break;
    }
    if (ksplit > 1) {
      a.ksplit = ksplit;
      a.grid = tiles * ksplit;
      cfg.gridDim = dim3(tiles * ksplit);
      attr[0].val.clusterDim.x = ksplit;
      cfg.numAttrs = g_opt_pdl ? 2 : 1;
      return cudaLaunchKernelEx(&cfg, gemm_tc_kernel<EPI, PAIR>, map_x, map_w, a) == cudaSuccess ? MDB_OK : MDB_ERR_CUDA;
    }
  }
  if (!PAIR)
    return mdb_launch(gemm_tc_kernel<EPI, PAIR>, dim3(tiles < sm_count ? tiles : sm_count), dim3(tc_threads(EPI)), kSmem,
                      st, map_x, map_w, a);
  // clusters of two CTAs, with programmatic dependent launch like every other kernel of the library
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sm_count / 2 * 2);
  cfg.blockDim = dim3(tc_threads(EPI));
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // CTA pairs the device holds at once (an odd SM of a processing cluster cannot host a pair)
  static int max_pairs = 0;
  if (max_pairs == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_kernel<EPI, PAIR>, &cfg) != cudaSuccess || n <= 0) n = sm_count / 2;
    max_pairs = n;
  }
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  cfg.gridDim = dim3(2 * pairs);
  a.grid = 2 * pairs;
  cfg.numAttrs = g_opt_pdl ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, gemm_tc_kernel<EPI, PAIR>, map_x, map_w, a) == cudaSuccess ? MDB_OK : MDB_ERR_CUDA;
}

// CTA pairs from 2048 rows on (measured: +12 .. 15 % on the bf16-store projections at 4096 and 16384 rows, even at
// 2048, where eight 256-row tiles per weight tile leave the pair form no room); MDB_OPT_GEMM_PAIR = 2 takes them
// from 256 rows, 0 never.
template <int EPI>
static int launch_tc(const bf16* x, int64_t ldx, const bf16* w, int w_rows, TcArgs& a, cudaStream_t st) {
  const int from_rows = g_opt_gemm_pair == 2 ? 2 * kTcBM : 2048;
  if (g_opt_gemm_pair != 0 && a.m >= from_rows) return launch_tc_impl<EPI, true>(x, ldx, w, w_rows, a, st);
  return launch_tc_impl<EPI, false>(x, ldx, w, w_rows, a, st);
}

}  // namespace mdb
