// Attention on the 5th-generation tensor cores, in two forms that share one
// warp-specialised pipeline:
//   * block attention over the paged KV cache (decode: the masked block of
//     every request against its committed prefix, every key visible;
//     flash_attn_with_kvcache as nanovllm/layers/sdar_attention.py:50-55 calls it);
//   * staircase attention over packed sequences (prefill: a query row sees the
//     keys up to the right edge of its right-aligned block;
//     nanovllm/kernels/triton/attention/block_prefill_attention_v2.py:17-166).
//
// One work unit = the query rows of `tokens x group` (tokens of one request or
// sequence times the query heads that share a KV head; row = token * group +
// head_in_group) against a key range.  ROWS = 64 or 128 rows per unit: the MMA
// is always M = 128.  With ROWS = 64 (paged form) the Q tile holds the rows
// twice, so that S carries every row in two tensor-memory lanes and the softmax
// of a tile is spread over four warps, two per row, 64 keys each; the P tile has
// the 64 real rows only (the upper operand rows of P V are whatever follows in
// shared memory and feed accumulator lanes nobody reads).  Persistent
// CTAs, one per SM, walk the units; inside a CTA
//   producer warp  TMA: the Q tile (3-D box: 64 channels x group x tokens) and
//            128-key K and V tiles ([tokens, hkv*128] seen as a matrix, boxes
//            of 128 rows x 64 channels, 128-byte swizzle) into K and V rings;
//   MMA warp       S = Q K^T (tcgen05.mma M128 N128, both operands K-major)
//            into one of two S buffers in tensor memory, one tile ahead of
//            O += P V (P from shared memory K-major, V as the MN-major B
//            operand: its rows are the K dimension);
//   softmax warps  one query row per thread: S read with tcgen05.ld, running
//            maximum kept lazily (O is rescaled only when a row's maximum
//            grows by more than 2^8, so the common tile needs no
//            read-modify-write of O), P rounded to bf16 into shared memory,
//            and at the end of the unit O/l to the output or the (max, sum,
//            O) partial to the split workspace.
// Tensor memory: S0 | S1 | O, 128 columns each.
//
// HBM traffic of the paged form is K and V once: 512 bytes per key per KV head.
#include "mdb_common.cuh"

namespace mdb {

constexpr int kAtKeys = 128;                          // keys per tile
constexpr int kAtHalfBytes = kAtKeys * 128;           // [128 keys][64 channels] bf16
constexpr int kAtTileBytes = 2 * kAtHalfBytes;        // 32 KB
constexpr float kAtRescaleStep = 8.0f;                // log2 units a row maximum may lag behind
constexpr int kAtMaxRanked = 512;                     // batches above this are walked in request order

// Shared-memory plan for ROWS query rows per unit (224 KB of tiles either way).
//
// DUP (64-row units of the paged form): the softmax of a 128-key tile is bound by the exponential unit of the
// sub-partitions that hold the softmax warps (128 ex2 per row on a quarter-rate pipe), so the 64 rows are spread
// over all four: the Q tile holds the 64 rows twice (operand rows 64..127 repeat rows 0..63), S = Q K^T therefore
// carries every row in two tensor-memory lanes, and the thread of lane r takes keys 0..63 of the tile while the
// thread of lane r + 64 takes keys 64..127 of the same row.  The two exchange their row maximum through shared
// memory, write their halves of the same P row, and add up their partial sums at the end of the unit.
template <int ROWS, bool DUP = false, bool STAIR = false>
struct AtPlan {
  static_assert(!DUP || ROWS == 64, "row duplication exists for the 64-row units");
  static constexpr int kQRows = DUP ? 128 : ROWS;     // rows of the Q operand tile
  static constexpr int kQBufs = (ROWS == 64 && !DUP) ? 2 : 1;
  // Staircase form: one P buffer is enough (the P V of a tile is long over when the next tile's softmax wants to
  // write), which buys the K ring a third stage: 4 x 4096 tokens 407 -> 396 us, one sequence of 16384 tokens
  // 1366 -> 1297 us.  (The paged form with 128-row units loses 3 % with the same trade and keeps two and two.)
  static constexpr int kPBufs = STAIR ? 1 : 2;
  static constexpr int kKStages = STAIR ? 3 : 2;
  static constexpr int kVStages = ROWS == 64 ? 3 : 2;
  static constexpr int kQBytes = 2 * kQRows * 128;    // two channel halves of [kQRows][128 B]
  static constexpr int kPBytes = 2 * ROWS * 128;      // two key halves of [ROWS][128 B]
  static constexpr int kSoftmaxWarps = DUP ? 4 : ROWS / 32;
  static constexpr int kCols = DUP ? 64 : 128;        // keys of a tile one softmax thread handles
  static constexpr int kProducerWarp = kSoftmaxWarps, kMmaWarp = kSoftmaxWarps + 1;
  static constexpr int kThreads = (kSoftmaxWarps + 2) * 32;
  static constexpr int kOffQ = 0;
  static constexpr int kOffP = kOffQ + kQBufs * kQBytes;
  static constexpr int kOffK = kOffP + kPBufs * kPBytes;
  static constexpr int kOffV = kOffK + kKStages * kAtTileBytes;
  static constexpr int kOffBars = kOffV + kVStages * kAtTileBytes;
  static constexpr int kMaxRanked = DUP ? 256 : kAtMaxRanked;          // batches above this are walked in request order
  static constexpr int kOffXch = kOffBars + 256 + 2 * kMaxRanked;   // DUP: [2][128] tagged values swapped by the two threads of a row
  // + barriers, tensor-memory slot, ranks; up to 1 KB in front to reach a 1024-byte boundary.  The DUP layout has
  // no room for that slack: it counts on the dynamic shared memory starting on such a boundary (it does when the
  // kernel has no static shared memory) and the kernel checks the size it was given before it touches anything.
  static constexpr int kSmemBytes = DUP ? kOffXch + 2 * 128 * 8 + 128 : 1024 + kOffXch;
};

// barrier slots (8 bytes each) after the tiles
enum {
  kAtBarQFull = 0, kAtBarQEmpty = 2, kAtBarKFull = 4, kAtBarKEmpty = 7, kAtBarVFull = 10, kAtBarVEmpty = 13,
  kAtBarSFull = 16, kAtBarSEmpty = 18, kAtBarPFull = 20, kAtBarPEmpty = 22, kAtBarOFull = 24, kAtBarOEmpty = 25,
  kAtBarQReady = 26, kAtBarCount = 28      // up to three K and three V stages
};

struct AtArgs {
  // common
  const bf16* q;
  bf16* out;
  int hq, hkv, group;
  int tokens_per_unit;      // tokens of one unit: ROWS / group, at most the block in the paged form
  float scale_log2;         // multiplies S before the softmax (1 in the staircase form: q is scaled instead)
  // paged form
  const int32_t* block_table;
  const int32_t* ctx_lens;
  float* part_o;            // [bs][nsplit][hq][block][128]
  float* part_ml;           // [bs][nsplit][hq][block][2]  (max in log2 units, sum)
  int table_stride, block, num_pages, nsplit, bs, row_blocks;
  // staircase form
  const int32_t* cu_seqlens;
  int64_t out_stride;
  int nseq, max_qtiles, log2_stairs;
  float q_scale;            // log2(e) / sqrt(D), applied to q and rounded to bf16 as the reference kernel does
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// 32 lanes x 32 consecutive fp32 columns
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
        "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])),
        "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
        "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])),
        "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])),
        "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }


// V tile as the B operand of O += P V: N = channels (contiguous, 64 per 128-byte
// row, the two channel halves kAtHalfBytes apart), K = keys (rows of 128 bytes,
// groups of 8 keys 1024 bytes apart).
__device__ __forceinline__ uint64_t umma_desc_sw128_mn(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>(kAtHalfBytes >> 4) << 16;          // leading byte offset: next 64 channels
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                  // stride byte offset: next 8 keys
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// The unit list every role walks the same way.
//
// Paged form: requests are ranked by context length (longest first; the ranks
// sit in shared memory) and the ranked units are dealt to the CTAs in
// alternating direction, wave by wave, so that every CTA gets about the same
// number of key tiles however ragged the batch is.
// Staircase form: units are (query tile, sequence, KV head) with the late
// (long) query tiles first.
struct AtUnit {
  bool valid;
  int ntiles;       // 128-key tiles
  int kbeg, kend;   // keys [kbeg, kend)
  int kvh;
  int q_tok0;       // row of the unit's first token in the q tensor
  int req, split, tok0;        // paged: request, key-range part, first token of the block covered
  bool ctx_clamped;            // paged: the context length exceeded what the page table can address
  int seq_start, m0, T;        // staircase: first packed row of the sequence, first token of the unit, length
};

template <bool STAIR>
__device__ __forceinline__ AtUnit at_unit(const AtArgs& a, const uint16_t* order, int units, int wave,
                                          int max_ranked = kAtMaxRanked) {
  AtUnit w = {};
  const int G = static_cast<int>(gridDim.x), c = static_cast<int>(blockIdx.x);
  if (STAIR) {
    const int p = wave * G + c;
    if (p >= units) return w;
    const int per_tile = a.nseq * a.hkv;
    const int qt = a.max_qtiles - 1 - p / per_tile;
    const int rest = p % per_tile;
    const int seq = rest / a.hkv;
    w.kvh = rest % a.hkv;
    w.seq_start = a.cu_seqlens[seq];
    w.T = a.cu_seqlens[seq + 1] - w.seq_start;
    w.m0 = qt * a.tokens_per_unit;
    if (w.m0 >= w.T) return w;
    w.valid = true;
    w.q_tok0 = w.seq_start + w.m0;
    const int S = 1 << a.log2_stairs;
    const int pad = ((w.T + S - 1) >> a.log2_stairs << a.log2_stairs) - w.T;
    const int last = min(w.m0 + a.tokens_per_unit, w.T) - 1;
    w.kbeg = 0;
    w.kend = min(w.T, ((((last + pad) >> a.log2_stairs) + 1) << a.log2_stairs) - pad);
    w.ntiles = (w.kend + kAtKeys - 1) / kAtKeys;
    return w;
  }
  const int p = wave * G + ((wave & 1) ? G - 1 - c : c);
  if (p >= units) return w;
  w.valid = true;
  const int per_req = a.hkv * a.row_blocks * a.nsplit;
  const int ranked = p / per_req, rem = p % per_req;
  w.req = a.bs <= max_ranked ? static_cast<int>(order[ranked]) : ranked;
  w.kvh = rem / (a.row_blocks * a.nsplit);
  w.tok0 = (rem / a.nsplit) % a.row_blocks * a.tokens_per_unit;
  w.split = rem % a.nsplit;
  w.q_tok0 = w.req * a.block + w.tok0;
  int ctx = a.ctx_lens[w.req];
  // A context longer than the page table's row can address is cut to the row (the producer warp raises
  // MDB_STATUS_BAD_PAGE for it): no role ever reads the table past the request's row.
  const int ctx_cap = a.table_stride * kPage;
  if (ctx > ctx_cap) { ctx = ctx_cap; w.ctx_clamped = true; }
  const int chunk = attn_part_keys(ctx, a.nsplit, kAtKeys);
  w.kbeg = w.split * chunk;
  w.kend = min(ctx, w.kbeg + chunk);
  w.ntiles = w.kend > w.kbeg ? (w.kend - w.kbeg + kAtKeys - 1) / kAtKeys : 0;
  return w;
}

// A ring position: stage index and the parity of the phase that stage is in.
struct AtRing {
  int stage = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void advance(int stages) {
    if (++stage == stages) { stage = 0; phase ^= 1; }
  }
};

// DUP layout: the two threads that share a query row (tensor-memory lanes r and r + 64, in different warps) swap
// one float.  Each writes (running number, value) as one 8-byte word into its slot of buffer `number & 1` and polls
// the partner's slot of the same buffer until it carries the same number; a thread starts swap n + 2 only after
// it has read the partner's word of swap n + 1, which the partner wrote after reading this thread's word of swap
// n, so two buffers are enough.  The wait is bounded like every other wait of the kernel.
__device__ __forceinline__ bool at_swap(volatile unsigned long long* xch, int lane_row, uint32_t number, float mine,
                                        float& other) {
  volatile unsigned long long* buf = xch + (number & 1u) * 128;
  buf[lane_row] = (static_cast<unsigned long long>(number) << 32) | __float_as_uint(mine);
  unsigned long long deadline = 0;
  for (uint32_t it = 0;; ++it) {
    const unsigned long long v = buf[lane_row ^ 64];
    if (static_cast<uint32_t>(v >> 32) == number) {
      other = __uint_as_float(static_cast<uint32_t>(v));
      return true;
    }
    if ((it & 1023u) == 1023u) {
      const unsigned long long now = global_timer_ns();
      if (deadline == 0) deadline = now + g_wait_limit_ns;
      else if (now > deadline) return false;
    }
  }
}

template <int ROWS, bool STAIR, bool DUP = false>
__global__ void __launch_bounds__(AtPlan<ROWS, DUP, STAIR>::kThreads, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const AtArgs a, const int units) {
  using P = AtPlan<ROWS, DUP, STAIR>;
  static_assert(!(DUP && STAIR), "row duplication is a paged-form layout");
  extern __shared__ __align__(1024) unsigned char at_smem_raw[];
  const uint32_t raw = smem_u32(at_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* gen_base = at_smem_raw + (base - raw);
  if (DUP) {
    uint32_t given;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(given));
    if ((base - raw) + static_cast<uint32_t>(P::kOffXch + 2 * 128 * 8) > given) {   // never on the boards this was built for
      if (threadIdx.x == 0) report_status(MDB_STATUS_LAYOUT);
      return;
    }
  }
  const uint32_t bars = base + P::kOffBars;
  auto bar = [&](int slot) { return bars + 8u * static_cast<uint32_t>(slot); };
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(gen_base + P::kOffBars + 8 * kAtBarCount);
  uint16_t* order = reinterpret_cast<uint16_t*>(gen_base + P::kOffBars + 256);
  const int waves = (units + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = a.group;
  const int rows_used = group * a.tokens_per_unit;      // <= ROWS

  if (threadIdx.x == 0) trace_event(30, 0);
  pdl_launch_dependents();
  if (!STAIR && a.bs <= P::kMaxRanked) {
    // context lengths are step inputs, not written by the kernels this one is chained to
    for (int r = threadIdx.x; r < a.bs; r += P::kThreads) {
      const int mine = a.ctx_lens[r];
      int rank = 0;
      for (int o = 0; o < a.bs; ++o) {
        const int other = a.ctx_lens[o];
        rank += (other > mine || (other == mine && o < r)) ? 1 : 0;
      }
      order[rank] = static_cast<uint16_t>(r);
    }
  }
  if (DUP) {
    unsigned long long* xz = reinterpret_cast<unsigned long long*>(gen_base + P::kOffXch);
    for (int i = threadIdx.x; i < 256; i += P::kThreads) xz[i] = 0ull;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < kAtBarCount; ++s) {
      const bool by_softmax = (s >= kAtBarSEmpty && s < kAtBarSEmpty + 2) || (s >= kAtBarPFull && s < kAtBarPFull + 2) ||
                              s == kAtBarOEmpty || s >= kAtBarQReady;
      mbar_init(bar(s), by_softmax ? P::kSoftmaxWarps : 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == P::kMmaWarp) {
    const uint32_t slot = smem_u32(const_cast<uint32_t*>(&misc[0]));
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = misc[0];
  const uint32_t tmem_o = tmem_base + 256;
  if (threadIdx.x == 0) trace_event(30, 1);
  pdl_wait();   // q and the K/V rows of this step come from the preceding kernel
  if (threadIdx.x == 0) trace_event(30, 2);

  if (warp == P::kProducerWarp) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      AtRing kr, vr, qr;
      uint32_t pend_k = 0, pend_v = 0, pend_q = 0;          // stages with a copy in flight, and the parity it completes
      uint32_t par_k = 0, par_v = 0, par_q = 0;
      bool ok = true;
      auto load_tile = [&](const CUtensorMap* map, uint32_t tiles0, int full0, int empty0, int stages, AtRing& r,
                           uint32_t& pend, uint32_t& par, int kvh, int token_row) {
        if (!mbar_wait(bar(empty0 + r.stage), r.phase ^ 1)) return false;
        const uint32_t full = bar(full0 + r.stage);
        const uint32_t dst = tiles0 + r.stage * kAtTileBytes;
        mbar_arrive_expect_tx(full, kAtTileBytes);
        tma_load_2d(dst, map, kvh * kHeadDim, token_row, full);
        tma_load_2d(dst + kAtHalfBytes, map, kvh * kHeadDim + 64, token_row, full);
        pend |= 1u << r.stage;
        par = (par & ~(1u << r.stage)) | (r.phase << r.stage);
        r.advance(stages);
        return true;
      };
      for (int wave = 0; wave < waves && ok; ++wave) {
        const AtUnit w = at_unit<STAIR>(a, order, units, wave, P::kMaxRanked);
        if (w.ctx_clamped) report_status(MDB_STATUS_BAD_PAGE);
        if (w.ntiles == 0) continue;
        if (!mbar_wait(bar(kAtBarQEmpty + qr.stage), qr.phase ^ 1)) { ok = false; break; }
        {
          const uint32_t full = bar(kAtBarQFull + qr.stage);
          const uint32_t dst = base + P::kOffQ + qr.stage * P::kQBytes;
          mbar_arrive_expect_tx(full, static_cast<uint32_t>(rows_used) * (DUP ? 512u : 256u));
          tma_load_3d(dst, &map_q, 0, w.kvh * group, w.q_tok0, full);
          tma_load_3d(dst + P::kQRows * 128, &map_q, 64, w.kvh * group, w.q_tok0, full);
          if (DUP) {      // the same rows once more as operand rows 64..
            tma_load_3d(dst + 64 * 128, &map_q, 0, w.kvh * group, w.q_tok0, full);
            tma_load_3d(dst + P::kQRows * 128 + 64 * 128, &map_q, 64, w.kvh * group, w.q_tok0, full);
          }
          pend_q |= 1u << qr.stage;
          par_q = (par_q & ~(1u << qr.stage)) | (qr.phase << qr.stage);
          qr.advance(P::kQBufs);
        }
        auto token_row = [&](int tile) {
          const int key0 = w.kbeg + tile * kAtKeys;
          if (STAIR) return w.seq_start + key0;
          int page = a.block_table[static_cast<int64_t>(w.req) * a.table_stride + key0 / kPage];
          if (page < 0 || page >= a.num_pages) {
            report_status(MDB_STATUS_BAD_PAGE);
            page = 0;
          }
          return page * kPage + key0 % kPage;
        };
        // in the order the MMA warp needs them: K0 K1 V0 K2 V1 ...
        for (int j = 0; j < w.ntiles && ok; ++j) {
          if (j == 0)
            ok = load_tile(&map_k, base + P::kOffK, kAtBarKFull, kAtBarKEmpty, P::kKStages, kr, pend_k, par_k, w.kvh, token_row(0));
          if (ok && j + 1 < w.ntiles)
            ok = load_tile(&map_k, base + P::kOffK, kAtBarKFull, kAtBarKEmpty, P::kKStages, kr, pend_k, par_k, w.kvh, token_row(j + 1));
          if (ok)
            ok = load_tile(&map_v, base + P::kOffV, kAtBarVFull, kAtBarVEmpty, P::kVStages, vr, pend_v, par_v, w.kvh, token_row(j));
        }
      }
      if (!ok) {
        report_status(MDB_STATUS_WAIT_TIMEOUT);
        // let the copies already issued land before the CTA gives its shared memory back
        for (int s = 0; s < P::kKStages; ++s) if (pend_k >> s & 1) mbar_wait(bar(kAtBarKFull + s), par_k >> s & 1);
        for (int s = 0; s < P::kVStages; ++s) if (pend_v >> s & 1) mbar_wait(bar(kAtBarVFull + s), par_v >> s & 1);
        for (int s = 0; s < P::kQBufs; ++s) if (pend_q >> s & 1) mbar_wait(bar(kAtBarQFull + s), par_q >> s & 1);
      }
    }
  } else if (warp == P::kMmaWarp) {
    // ----------------------------------------------------------------- MMA issue
    // All 32 lanes walk the loops with warp-uniform operands and one elected lane issues each tcgen05
    // instruction: issued from a single lane of a divergent warp every tcgen05.mma costs ~130 cycles of issue
    // time, which at 16 instructions per key tile is twice the time the tensor pipe needs for them.
    {
      // bf16 x bf16 -> fp32, M = 128, N = 128; bit 16 set: B operand MN-major
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kAtKeys >> 3) << 17) |
                               (static_cast<uint32_t>(128 >> 4) << 24);
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                               (static_cast<uint32_t>(kHeadDim >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
      AtRing kr, vr, qr, sr, pr;        // sr: S buffer the next S = Q K^T goes to; pr: P buffer of the next P V
      uint32_t o_phase = 0;             // parity of the o_empty phase to wait for
      bool ok = true;
      for (int wave = 0; wave < waves && ok; ++wave) {
        const AtUnit w = at_unit<STAIR>(a, order, units, wave, P::kMaxRanked);
        if (w.ntiles == 0) continue;
        // staircase form: the softmax warps scale q in place first
        if (!mbar_wait_w(bar((STAIR ? kAtBarQReady : kAtBarQFull) + qr.stage), qr.phase)) { ok = false; break; }
        const uint32_t q_tile = base + P::kOffQ + qr.stage * P::kQBytes;
        auto issue_s = [&](int j) {
          if (!mbar_wait_w(bar(kAtBarKFull + kr.stage), kr.phase)) return false;
          if (!mbar_wait_w(bar(kAtBarSEmpty + sr.stage), sr.phase ^ 1)) return false;
          tc_fence_after();
          const uint32_t k_tile = base + P::kOffK + kr.stage * kAtTileBytes;
          const uint32_t d_tmem = tmem_base + sr.stage * kAtKeys;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t adesc = umma_desc_sw128(q_tile + (kk >> 2) * (P::kQRows * 128)) + 2 * (kk & 3);
            const uint64_t bdesc = umma_desc_sw128(k_tile + (kk >> 2) * kAtHalfBytes) + 2 * (kk & 3);
            umma_bf16_w(d_tmem, adesc, bdesc, idesc_s, kk > 0 ? 1u : 0u);
          }
          umma_commit_w(bar(kAtBarKEmpty + kr.stage));
          umma_commit_w(bar(kAtBarSFull + sr.stage));
          if (j == w.ntiles - 1) umma_commit_w(bar(kAtBarQEmpty + qr.stage));
          kr.advance(P::kKStages);
          sr.advance(2);
          return true;
        };
        ok = issue_s(0);
        for (int j = 0; j < w.ntiles && ok; ++j) {
          if (j + 1 < w.ntiles) ok = issue_s(j + 1);
          if (!ok) break;
          if (!mbar_wait_w(bar(kAtBarVFull + vr.stage), vr.phase)) { ok = false; break; }
          if (!mbar_wait_w(bar(kAtBarPFull + pr.stage), pr.phase)) { ok = false; break; }
          if (j == 0) {
            // the previous unit's accumulator must have been read out
            if (!mbar_wait_w(bar(kAtBarOEmpty), o_phase ^ 1)) { ok = false; break; }
            o_phase ^= 1;
          }
          tc_fence_after();
          const uint32_t p_tile = base + P::kOffP + pr.stage * P::kPBytes;
          const uint32_t v_tile = base + P::kOffV + vr.stage * kAtTileBytes;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t adesc = umma_desc_sw128(p_tile + (kk >> 2) * (ROWS * 128)) + 2 * (kk & 3);
            const uint64_t bdesc = umma_desc_sw128_mn(v_tile + kk * 2048);
            umma_bf16_w(tmem_o, adesc, bdesc, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit_w(bar(kAtBarVEmpty + vr.stage));
          umma_commit_w(bar(kAtBarPEmpty + pr.stage));
          if (j == w.ntiles - 1) umma_commit_w(bar(kAtBarOFull));
          vr.advance(P::kVStages);
          pr.advance(P::kPBufs);
        }
        qr.advance(P::kQBufs);
      }
      if (!ok && lane == 0) report_status(MDB_STATUS_WAIT_TIMEOUT);
    }
  } else {
    // ------------------------------------------------------------------- softmax
    const int lane_row = 32 * warp + lane;                 // tensor-memory lane of this thread
    const int row = DUP ? (lane_row & 63) : lane_row;      // query row of the unit
    const int half = DUP ? (lane_row >> 6) : 0;            // DUP: which 64 keys of a tile this thread takes
    const int col0 = 64 * half;
    constexpr int NC = P::kCols;
    const int tok_local = row / group, head_in_group = row % group;
    const uint32_t lane_field = static_cast<uint32_t>(32 * warp) << 16;
    volatile unsigned long long* xch = reinterpret_cast<volatile unsigned long long*>(gen_base + P::kOffXch);
    uint32_t xseq = 0;                                     // DUP: running number of the swaps of this thread
    AtRing sr, pr, vr, qr;             // positions of the tile being handled in the S, P, V and Q rings
    uint32_t prev_p_stage = 0, prev_p_phase = 0;   // P ring position of the previous tile (its P V frees O for a rescale)
    uint32_t o_phase = 0;
    bool ok = true;
    for (int wave = 0; wave < waves && ok; ++wave) {
      const AtUnit w = at_unit<STAIR>(a, order, units, wave, P::kMaxRanked);
      if (!w.valid) continue;
      const int head = w.kvh * group + head_in_group;
      bool row_valid = row < rows_used;
      int limit = 0;                 // staircase form: last key this row sees
      bf16* out_row;
      int64_t prow = 0;
      if (STAIR) {
        const int i = w.m0 + tok_local;
        row_valid = row_valid && i < w.T;
        const int S = 1 << a.log2_stairs;
        const int pad = ((w.T + S - 1) >> a.log2_stairs << a.log2_stairs) - w.T;
        limit = row_valid ? min(w.T - 1, ((((i + pad) >> a.log2_stairs) + 1) << a.log2_stairs) - 1 - pad) : -1;
        out_row = a.out + static_cast<int64_t>(w.seq_start + (row_valid ? i : 0)) * a.out_stride + head * kHeadDim;
      } else {
        const int tok = w.tok0 + tok_local;
        row_valid = row_valid && tok < a.block;
        const int tk = row_valid ? tok : 0;
        prow = ((static_cast<int64_t>(w.req) * a.nsplit + w.split) * a.hq + head) * a.block + tk;
        out_row = a.out + ((static_cast<int64_t>(w.req) * a.block + tk) * a.hq + head) * kHeadDim;
      }
      if (w.ntiles == 0) {           // paged form only: an empty key range
        if (row_valid && half == 0) {
          if (a.nsplit == 1) {
#pragma unroll
            for (int c = 0; c < 16; ++c) reinterpret_cast<uint4*>(out_row)[c] = make_uint4(0u, 0u, 0u, 0u);
          } else {
            float4* po = reinterpret_cast<float4*>(a.part_o + prow * kHeadDim);
#pragma unroll
            for (int c = 0; c < 32; ++c) po[c] = make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float2*>(a.part_ml + prow * 2) = make_float2(-INFINITY, 0.f);
          }
        }
        continue;
      }
      if (STAIR) {
        // q * log2(e)/sqrt(D) rounded to bf16, in place (elementwise, so the swizzle does not matter)
        ok = mbar_wait(bar(kAtBarQFull + qr.stage), qr.phase);
        if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
        if (row < rows_used) {
          const uint32_t q_row = base + P::kOffQ + qr.stage * P::kQBytes + row * 128;
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const uint32_t addr = q_row + (c >> 3) * (ROWS * 128) + (c & 7) * 16;
            uint32_t x[4];
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x[0]), "=r"(x[1]), "=r"(x[2]), "=r"(x[3]) : "r"(addr));
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = unpack_bf16x2(x[e]);
              x[e] = pack_bf16x2(f.x * a.q_scale, f.y * a.q_scale);
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x[0]), "r"(x[1]), "r"(x[2]), "r"(x[3]) : "memory");
          }
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(kAtBarQReady + qr.stage));
        qr.advance(P::kQBufs);
      }
      float m_ref = -INFINITY, l = 0.f;
      for (int j = 0; j < w.ntiles; ++j) {
        ok = mbar_wait(bar(kAtBarSFull + sr.stage), sr.phase);
        if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
        tc_fence_after();
        const uint32_t s_addr = tmem_base + sr.stage * kAtKeys + lane_field;
        const int key0 = w.kbeg + j * kAtKeys;
        // keys of this tile the row sees: [0, nvalid)
        const int nvalid = STAIR ? max(0, min(kAtKeys, limit + 1 - key0)) : min(kAtKeys, w.kend - key0);
        // the thread's share of the score row into registers, then the S buffer goes back to the MMA warp
        float s[NC];
#pragma unroll
        for (int c = 0; c < NC / 32; ++c) tmem_ld32(s_addr + col0 + 32 * c, s + 32 * c);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(kAtBarSEmpty + sr.stage));
        const int nv = nvalid - col0;               // valid keys among this thread's columns: [0, nv)
        if (nv < NC) {
#pragma unroll
          for (int i = 0; i < NC; ++i) if (i >= nv) s[i] = -INFINITY;   // also replaces NaN from stale rows
        }
        // eight independent chains: the warp is alone on its sub-partition, nothing else hides the ALU latency
        float mxv[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) mxv[k] = s[k];
#pragma unroll
        for (int i = 8; i < NC; i += 8) {
#pragma unroll
          for (int k = 0; k < 8; ++k) mxv[k] = fmaxf(mxv[k], s[i + k]);
        }
        float mx = fmaxf(fmaxf(fmaxf(mxv[0], mxv[1]), fmaxf(mxv[2], mxv[3])), fmaxf(fmaxf(mxv[4], mxv[5]), fmaxf(mxv[6], mxv[7])));
        if (DUP) {
          // the other half of the row's keys is with the thread 64 lanes away (two warps further): swap maxima
          float other;
          ok = at_swap(xch, lane_row, ++xseq, mx, other);
          if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
          mx = fmaxf(mx, other);
        }
        if (!row_valid) mx = 0.f;                             // rows past the block hold whatever the tile held
        const float m_tile = mx * a.scale_log2;
        // a row that sees no key of this tile (staircase form, rows above the tile's diagonal) keeps its state
        const bool grow = m_tile > m_ref + kAtRescaleStep || (m_ref == -INFINITY && m_tile != -INFINITY);
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = fmaxf(m_ref, m_tile);
          const float f = m_ref == -INFINITY ? 0.f : ex2_approx(m_ref - m_new);
          l *= f;
          if (j > 0 && half == 0) {     // (DUP: the rows' accumulators are read from lanes 0..63, whose threads rescale them)
            // O is quiet once the previous tile's P V has completed
            ok = mbar_wait(bar(kAtBarPEmpty + prev_p_stage), prev_p_phase);
            if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              float o[32];
              tmem_ld32(tmem_o + lane_field + 32 * c, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] *= f;
              tmem_st32(tmem_o + lane_field + 32 * c, o);
            }
            tmem_st_wait();
          }
          m_ref = m_new;
        }
        // P = 2^(s * scale - m_ref) rounded to bf16; a masked key gives 2^-inf = 0
        const float m_use = m_ref == -INFINITY ? 0.f : m_ref;   // nothing seen yet: every s is -inf, P = 0
        uint32_t pk[NC / 2];
        float lv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < NC; i += 8) {
          float pv[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) pv[k] = ex2_approx(fmaf(s[i + k], a.scale_log2, -m_use));
#pragma unroll
          for (int k = 0; k < 8; ++k) lv[k] += pv[k];
#pragma unroll
          for (int k = 0; k < 8; k += 2) pk[(i + k) >> 1] = pack_bf16x2(pv[k], pv[k + 1]);
        }
        l += ((lv[0] + lv[1]) + (lv[2] + lv[3])) + ((lv[4] + lv[5]) + (lv[6] + lv[7]));
        // the P buffer of this tile is free once the P V two tiles back has completed
        ok = mbar_wait(bar(kAtBarPEmpty + pr.stage), pr.phase ^ 1);
        if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
        // K-major swizzled P tile: 16-byte chunk q of key half h holds keys 64 h + 8 q .. + 7
        const uint32_t p_row = base + P::kOffP + pr.stage * P::kPBytes + row * 128;
#pragma unroll
        for (int q = 0; q < NC / 8; ++q) {
          const uint32_t chunk = static_cast<uint32_t>(q & 7) ^ static_cast<uint32_t>(row & 7);
          const int key_half = DUP ? half : (q >> 3);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(p_row + key_half * (ROWS * 128) + (chunk << 4)),
                       "r"(pk[4 * q]), "r"(pk[4 * q + 1]), "r"(pk[4 * q + 2]), "r"(pk[4 * q + 3])
                       : "memory");
        }
        if (!STAIR && nvalid < kAtKeys) {
          // stale cache rows past the context end must not reach O through 0 * (Inf or NaN): clear them in V
          ok = mbar_wait(bar(kAtBarVFull + vr.stage), vr.phase);
          if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
          const uint32_t v_tile = base + P::kOffV + vr.stage * kAtTileBytes;
          for (int r = nvalid + lane_row; r < kAtKeys; r += 32 * P::kSoftmaxWarps) {
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
              for (int c = 0; c < 8; ++c)
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(v_tile + h * kAtHalfBytes + r * 128 + c * 16),
                             "r"(0u)
                             : "memory");
          }
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(kAtBarPFull + pr.stage));
        prev_p_stage = pr.stage;
        prev_p_phase = pr.phase;
        sr.advance(2);
        pr.advance(P::kPBufs);
        vr.advance(P::kVStages);
      }
      if (!ok) break;
      // ------------------------------------------------------------- unit epilogue
      ok = mbar_wait(bar(kAtBarOFull), o_phase);
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      o_phase ^= 1;
      tc_fence_after();
      if (DUP) {                       // the row's sum of probabilities: this thread's keys + the partner's
        float other;
        ok = at_swap(xch, lane_row, ++xseq, l, other);
        if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
        l += other;
      }
      if (half != 0) {
        // DUP: lanes 64..127 of O belong to operand rows nobody wrote; the rows' outputs leave from lanes 0..63
      } else if (STAIR || a.nsplit == 1) {
        const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          float o[32];
          tmem_ld32(tmem_o + lane_field + 32 * c, o);
          tmem_ld_wait();
          if (row_valid) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
              reinterpret_cast<uint4*>(out_row + 32 * c)[q4] =
                  make_uint4(pack_bf16x2(o[8 * q4] * inv, o[8 * q4 + 1] * inv), pack_bf16x2(o[8 * q4 + 2] * inv, o[8 * q4 + 3] * inv),
                             pack_bf16x2(o[8 * q4 + 4] * inv, o[8 * q4 + 5] * inv), pack_bf16x2(o[8 * q4 + 6] * inv, o[8 * q4 + 7] * inv));
          }
        }
      } else {
        float4* po = reinterpret_cast<float4*>(a.part_o + prow * kHeadDim);
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          float o[32];
          tmem_ld32(tmem_o + lane_field + 32 * c, o);
          tmem_ld_wait();
          if (row_valid) {
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4) po[8 * c + q4] = make_float4(o[4 * q4], o[4 * q4 + 1], o[4 * q4 + 2], o[4 * q4 + 3]);
          }
        }
        if (row_valid) *reinterpret_cast<float2*>(a.part_ml + prow * 2) = make_float2(m_ref, l);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kAtBarOEmpty));
    }
    if (!ok && lane == 0) report_status(MDB_STATUS_WAIT_TIMEOUT);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == P::kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---- host side ---------------------------------------------------------------
struct QMapKey {
  const void* ptr;
  int64_t tokens, row_stride;
  int hq, group, box_tokens;
  bool operator==(const QMapKey& o) const {
    return ptr == o.ptr && tokens == o.tokens && row_stride == o.row_stride && hq == o.hq && group == o.group &&
           box_tokens == o.box_tokens;
  }
};
struct QMapKeyHash {
  size_t operator()(const QMapKey& k) const {
    return reinterpret_cast<size_t>(k.ptr) ^ static_cast<size_t>(k.tokens) * 0x9e3779b97f4a7c15ull ^
           static_cast<size_t>(k.row_stride) * 0xc2b2ae3d27d4eb4full ^
           static_cast<size_t>(k.hq * 131 + k.group * 17 + k.box_tokens);
  }
};

// Tensor map of q [tokens, hq, 128] bf16 (token stride row_stride elements) read in boxes of
// 64 channels x group heads x box_tokens tokens.
static bool get_q_tensor_map(const void* ptr, int64_t tokens, int64_t row_stride, int hq, int group, int box_tokens,
                             CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<QMapKey, CUtensorMap, QMapKeyHash> cache;
  const QMapKey key{ptr, tokens, row_stride, hq, group, box_tokens};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return true;
  }
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return false;
  CUtensorMap m;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(kHeadDim), static_cast<cuuint64_t>(hq), static_cast<cuuint64_t>(tokens)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(kHeadDim) * 2, static_cast<cuuint64_t>(row_stride) * 2};
  const cuuint32_t box[3] = {64u, static_cast<cuuint32_t>(group), static_cast<cuuint32_t>(box_tokens)};
  const cuuint32_t estr[3] = {1, 1, 1};
  if (enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 1024) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return true;
}

static int at_sm_count() {
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  return sm_count;
}

template <int ROWS, bool STAIR, bool DUP = false>
static int at_launch(const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v, const AtArgs& a,
                     int64_t units, cudaStream_t st) {
  using P = AtPlan<ROWS, DUP, STAIR>;
  static PerDeviceOnce attr_once;
  const int dev = attr_once.slot();
  if (dev < 0) return MDB_ERR_CUDA;
  if (!attr_once.done[dev]) {
    if (cudaFuncSetAttribute(attn_tc_kernel<ROWS, STAIR, DUP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             P::kSmemBytes) != cudaSuccess)
      return MDB_ERR_CUDA;
    attr_once.done[dev] = true;
  }
  if (units > (1 << 30)) return MDB_ERR_UNSUPPORTED;
  const int sms = at_sm_count();
  const int grid = units < sms ? static_cast<int>(units) : sms;
  return mdb_launch(attn_tc_kernel<ROWS, STAIR, DUP>, dim3(grid), dim3(P::kThreads), P::kSmemBytes, st, map_q, map_k,
                    map_v, a, static_cast<int>(units));
}

// ---- paged form ----
static bool attn_tc_supported(int block, int hq, int hkv, float softmax_scale) {
  if (hkv <= 0 || hq % hkv != 0) return false;
  const int group = hq / hkv;
  return group <= 128 && block >= 1 && block <= 256 && softmax_scale > 0.f;
}

static int attn_tc_launch(const AttnPagedArgs& pa, int bs, cudaStream_t st) {
  AtArgs a = {};
  a.q = pa.q;
  a.out = pa.out;
  a.hq = pa.hq; a.hkv = pa.hkv; a.group = pa.hq / pa.hkv;
  a.scale_log2 = pa.scale_log2;
  a.block_table = pa.block_table;
  a.ctx_lens = pa.ctx_lens;
  a.part_o = pa.part_o;
  a.part_ml = pa.part_ml;
  a.table_stride = pa.table_stride;
  a.block = pa.block;
  a.num_pages = pa.num_pages;
  a.nsplit = pa.nsplit;
  a.bs = bs;
  const int rows = a.group * pa.block <= 64 ? 64 : 128;
  a.tokens_per_unit = rows / a.group < pa.block ? rows / a.group : pa.block;
  a.row_blocks = (pa.block + a.tokens_per_unit - 1) / a.tokens_per_unit;
  CUtensorMap map_q, map_k, map_v;
  const int64_t cache_rows = static_cast<int64_t>(pa.num_pages) * kPage;
  if (!get_q_tensor_map(pa.q, static_cast<int64_t>(bs) * pa.block, static_cast<int64_t>(pa.hq) * kHeadDim, pa.hq, a.group,
                        a.tokens_per_unit, &map_q))
    return MDB_ERR_CUDA;
  if (!get_tensor_map(pa.k_cache, cache_rows, pa.hkv * kHeadDim, pa.hkv * kHeadDim, kAtKeys, &map_k)) return MDB_ERR_CUDA;
  if (!get_tensor_map(pa.v_cache, cache_rows, pa.hkv * kHeadDim, pa.hkv * kHeadDim, kAtKeys, &map_v)) return MDB_ERR_CUDA;
  const int64_t units = static_cast<int64_t>(bs) * pa.hkv * a.row_blocks * pa.nsplit;
  return rows == 64 ? at_launch<64, false, true>(map_q, map_k, map_v, a, units, st)
                    : at_launch<128, false>(map_q, map_k, map_v, a, units, st);
}

// ---- staircase form ----
static bool attn_stair_tc_supported(int hq, int hkv, int64_t q_stride, int64_t k_stride, int64_t v_stride) {
  if (hkv <= 0 || hq % hkv != 0 || hq / hkv > 128) return false;
  return q_stride % 8 == 0 && k_stride % 8 == 0 && v_stride % 8 == 0;
}

static int attn_stair_tc_launch(const AttnStairArgs& sa, int nseq, int max_seqlen, int64_t total_tokens, cudaStream_t st) {
  AtArgs a = {};
  a.q = sa.q;
  a.out = sa.out;
  a.hq = sa.hq; a.hkv = sa.hkv; a.group = sa.hq / sa.hkv;
  a.scale_log2 = 1.0f;
  a.q_scale = sa.q_scale;
  a.cu_seqlens = sa.cu_seqlens;
  a.out_stride = sa.out_stride;
  a.nseq = nseq;
  a.log2_stairs = sa.log2_stairs;
  a.tokens_per_unit = 128 / a.group;
  a.max_qtiles = (max_seqlen + a.tokens_per_unit - 1) / a.tokens_per_unit;
  a.nsplit = 1;
  CUtensorMap map_q, map_k, map_v;
  if (!get_q_tensor_map(sa.q, total_tokens, sa.q_stride, sa.hq, a.group, a.tokens_per_unit, &map_q)) return MDB_ERR_CUDA;
  if (!get_tensor_map(sa.k, total_tokens, sa.hkv * kHeadDim, sa.k_stride, kAtKeys, &map_k)) return MDB_ERR_CUDA;
  if (!get_tensor_map(sa.v, total_tokens, sa.hkv * kHeadDim, sa.v_stride, kAtKeys, &map_v)) return MDB_ERR_CUDA;
  const int64_t units = static_cast<int64_t>(a.max_qtiles) * nseq * sa.hkv;
  return at_launch<128, true>(map_q, map_k, map_v, a, units, st);
}

}  // namespace mdb
