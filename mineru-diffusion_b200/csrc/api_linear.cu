// C entry points of the linear layers and the LM-head sampler: the weight-streaming
// kernel for steps of at most 64 rows, the tile GEMM for everything else.
#include "mdb_common.cuh"

using namespace mdb;

namespace {

int64_t align256(int64_t v) { return (v + 255) / 256 * 256; }

struct LmHeadLayout {
  int64_t nparts, off_i, off_logits, total;
};

LmHeadLayout lmhead_layout(int m, int vocab) {
  LmHeadLayout l;
  const bool streaming = m <= 64 && vocab % kWsTileRows == 0;   // weight-streaming kernel: one record per 128-column tile
  l.nparts = streaming ? vocab / kWsTileRows : (vocab + kTcBN - 1) / kTcBN;   // tile GEMM: one record per 256-column tile
  l.off_i = align256(l.nparts * m * 16);
  l.off_logits = l.off_i + align256(l.nparts * m * 4);
  l.total = l.off_logits + (streaming ? 0 : align256(static_cast<int64_t>(m) * vocab * 2));
  return l;
}

int finalize_sampler(const float4* part_f, const int* part_i, int nparts, int m, int32_t* x0_out, float* conf_out,
                     cudaStream_t st, const TpSignal tp = TpSignal{nullptr, nullptr, 0, 0, nullptr}) {
  return mdb_launch(sampler_finalize_kernel, dim3(m), dim3(kFinalizeThreads), 0, st, part_f, part_i, nparts, m, x0_out,
                    conf_out, tp);
}

int scan_logits(const bf16* logits, int64_t ld, int m, int vocab, const float* temperatures, int block, int noise_mode,
                const float* noise, uint32_t seed, uint32_t step, const uint32_t* step_dev, unsigned char* ws,
                int32_t* x0_out, float* conf_out, cudaStream_t st) {
  const int nparts = (vocab + kScanCols - 1) / kScanCols;
  float4* part_f = reinterpret_cast<float4*>(ws);
  int* part_i = reinterpret_cast<int*>(ws + align256(static_cast<int64_t>(nparts) * m * 16));
  dim3 grid(nparts, m);
  int rc = mdb_launch(logits_scan_kernel, grid, dim3(256), 0, st, logits, ld, m, vocab, temperatures, block, noise_mode,
                      noise, seed, step, step_dev, part_f, part_i);
  if (rc != MDB_OK) return rc;
  return finalize_sampler(part_f, part_i, nparts, m, x0_out, conf_out, st);
}

// k slices of the tensor-core streaming kernel: about one task per SM, at least four 64-wide chunks per slice
int ws_pick_ksplit(int n, int k) {
  const int tiles = n / kWsTileRows;
  const int chunks = k / kWsBK;
  int s = tiles > 0 ? 148 / tiles : 1;
  if (s < 1) s = 1;
  if (s > chunks / 4) s = chunks / 4 > 0 ? chunks / 4 : 1;
  if (s > 32) s = 32;
  // every slice must be non-empty
  while (s > 1 && ((chunks + s - 1) / s) * (s - 1) >= chunks) --s;
  return s;
}

// Common argument checks of the short-step entry points (at most 64 rows; 256 for the split-k slice form).
int check_short_step(const void* x, int64_t ldx, const void* w, int m, int n, int k, int max_rows = kWsMaxRows) {
  MDB_REQUIRE(x && w, MDB_ERR_ARG);
  MDB_REQUIRE(m >= 1 && m <= max_rows, MDB_ERR_UNSUPPORTED);
  MDB_REQUIRE(n > 0 && k > 0 && ldx >= k, MDB_ERR_ARG);
  MDB_REQUIRE(ldx % 8 == 0 && mdb_aligned16(x) && mdb_aligned16(w), MDB_ERR_ALIGN);
  return MDB_OK;
}

}  // namespace

extern "C" {

int mdb_gemm_pick_ksplit(int m, int n, int k) {
  if (m < 1 || n < 1 || k < 1 || !ws_supported(kWsPartial, m, n, k, k)) return 1;
  return ws_pick_ksplit(n, k);
}

int64_t mdb_gemm_splitk_workspace_bytes(int m, int n, int ksplit) {
  if (m <= 0 || n <= 0 || ksplit <= 0) return 0;
  return static_cast<int64_t>(ksplit) * m * n * 4;
}

int mdb_gemm_splitk_partials(const void* x, int64_t ldx, const void* w, float* partials, int m, int n, int k,
                             int ksplit, mdb_stream_t stream) {
  if (m == 0) return MDB_OK;
  int rc = check_short_step(x, ldx, w, m, n, k, kWsMaxRowsPartial);
  if (rc != MDB_OK) return rc;
  MDB_REQUIRE(partials != nullptr && ksplit >= 1 && ksplit <= 64, MDB_ERR_ARG);
  MDB_REQUIRE(mdb_aligned16(partials), MDB_ERR_ALIGN);
  MDB_REQUIRE(ws_supported(kWsPartial, m, n, k, ldx), MDB_ERR_UNSUPPORTED);
  const int chunks = k / kWsBK;
  const int per = (chunks + ksplit - 1) / ksplit;
  MDB_REQUIRE(per * (ksplit - 1) < chunks, MDB_ERR_ARG);   // no empty slice: every partial row is written
  WsArgs a = {};
  a.m = m; a.n = n; a.k = k; a.ksplit = ksplit;
  a.partials = partials;
  return launch_ws<kWsPartial>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(w), a,
                               static_cast<cudaStream_t>(stream));
}

int mdb_gemm_gateup_swiglu(const void* x, int64_t ldx, const void* w_gate_up, void* act, int64_t ld_act, int m,
                           int inter, int k, mdb_stream_t stream) {
  if (m == 0) return MDB_OK;
  MDB_REQUIRE(x && w_gate_up && act && m > 0 && inter > 0 && k > 0 && ldx >= k && ld_act >= inter, MDB_ERR_ARG);
  MDB_REQUIRE(ldx % 8 == 0 && ld_act % 2 == 0 && mdb_aligned16(x) && mdb_aligned16(w_gate_up) && mdb_aligned16(act),
              MDB_ERR_ALIGN);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ws_supported(kWsSwiglu, m, 2 * inter, k, ldx)) {
    // short step: the weight is streamed once, tiles of 64 gate rows + their 64 up rows
    WsArgs a = {};
    a.m = m; a.n = 2 * inter; a.k = k; a.ksplit = 1;
    a.inter = inter;
    a.y = static_cast<bf16*>(act);
    a.ldy = ld_act;
    return launch_ws<kWsSwiglu>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(w_gate_up), a, st);
  }
  // many rows: tile GEMM whose weight tile pairs 128 gate rows with their 128 up rows
  MDB_REQUIRE(tc_supported(kTcSwiglu, m, inter, k, ldx, ld_act), MDB_ERR_UNSUPPORTED);
  TcArgs a = {};
  a.m = m; a.n = inter; a.k = k; a.inter = inter;
  a.y = static_cast<bf16*>(act);
  a.ldy = ld_act;
  return launch_tc<kTcSwiglu>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(w_gate_up), 2 * inter, a, st);
}

int mdb_gemm_bf16(const void* x, int64_t ldx, const void* w, void* y, int64_t ldy, int m, int n, int k,
                  mdb_stream_t stream) {
  MDB_REQUIRE(m >= 0 && n > 0 && k > 0, MDB_ERR_ARG);
  if (m == 0) return MDB_OK;
  MDB_REQUIRE(x && w && y && ldx >= k && ldy >= n, MDB_ERR_ARG);
  MDB_REQUIRE(ldx % 8 == 0 && ldy % 2 == 0 && mdb_aligned16(x) && mdb_aligned16(w) && mdb_aligned16(y),
              MDB_ERR_ALIGN);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ws_supported(kWsBf16, m, n, k, ldx)) {
    WsArgs a = {};
    a.m = m; a.n = n; a.k = k; a.ksplit = 1;
    a.y = static_cast<bf16*>(y);
    a.ldy = ldy;
    return launch_ws<kWsBf16>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(w), a, st);
  }
  MDB_REQUIRE(tc_supported(kTcBf16, m, n, k, ldx, ldy), MDB_ERR_UNSUPPORTED);
  TcArgs a = {};
  a.m = m; a.n = n; a.k = k;
  a.y = static_cast<bf16*>(y);
  a.ldy = ldy;
  return launch_tc<kTcBf16>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(w), n, a, st);
}

int mdb_gemm_bf16_tp(const void* x, int64_t ldx, const void* w, void* y, void* y_peer, int64_t ldy, int m, int n, int k,
                     uint32_t* peer_flags, uint32_t tag, const uint32_t* epoch, int* grid_out, mdb_stream_t stream) {
  MDB_REQUIRE(m > 64 && n > 0 && k > 0, MDB_ERR_UNSUPPORTED);
  MDB_REQUIRE(x && w && y && y_peer && peer_flags && epoch && grid_out && ldx >= k && ldy >= n, MDB_ERR_ARG);
  MDB_REQUIRE(tag >= 1 && tag <= 255, MDB_ERR_ARG);
  MDB_REQUIRE(ldx % 8 == 0 && ldy % 8 == 0 && mdb_aligned16(x) && mdb_aligned16(w) && mdb_aligned16(y) &&
                  mdb_aligned16(y_peer),
              MDB_ERR_ALIGN);
  MDB_REQUIRE(tc_supported(kTcBf16, m, n, k, ldx, ldy), MDB_ERR_UNSUPPORTED);
  TcArgs a = {};
  a.m = m; a.n = n; a.k = k;
  a.y = static_cast<bf16*>(y);
  a.y_peer = static_cast<bf16*>(y_peer);
  a.ldy = ldy;
  a.tp = {peer_flags, nullptr, 0, tag, epoch};
  const int rc = launch_tc<kTcBf16>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(w), n, a,
                                    static_cast<cudaStream_t>(stream));
  *grid_out = a.grid;
  return rc;
}

int mdb_gemm_qkv_rope_commit(const void* x, int64_t ldx, const void* w_qkv, int m, int k, const int64_t* positions,
                             const float* rope_table, int max_pos, const void* q_norm_w, const void* k_norm_w,
                             float eps, const int32_t* slot_mapping, void* q_out, void* k_out, void* v_out,
                             void* k_cache, void* v_cache, int64_t num_slots, int hq, int hkv, mdb_stream_t stream) {
  MDB_REQUIRE(m >= 0 && k > 0 && hq > 0 && hkv > 0 && max_pos > 0, MDB_ERR_ARG);
  if (m == 0) return MDB_OK;
  MDB_REQUIRE(x && w_qkv && positions && rope_table && q_norm_w && k_norm_w && q_out && ldx >= k, MDB_ERR_ARG);
  MDB_REQUIRE(slot_mapping == nullptr || (k_cache && v_cache && num_slots > 0), MDB_ERR_ARG);
  MDB_REQUIRE(mdb_aligned16(x) && mdb_aligned16(w_qkv) && mdb_aligned16(rope_table) && mdb_aligned16(q_out) &&
                  mdb_aligned16(k_out) && mdb_aligned16(v_out) && mdb_aligned16(k_cache) && mdb_aligned16(v_cache) &&
                  mdb_aligned16(q_norm_w) && mdb_aligned16(k_norm_w),
              MDB_ERR_ALIGN);
  const int n = (hq + 2 * hkv) * kHeadDim;
  MDB_REQUIRE(tc_supported(kTcQkvRope, m, n, k, ldx, 0), MDB_ERR_UNSUPPORTED);
  TcArgs a = {};
  a.m = m; a.n = n; a.k = k;
  a.hq = hq; a.hkv = hkv; a.max_pos = max_pos;
  a.eps = eps;
  a.positions = positions;
  a.rope_table = rope_table;
  a.q_norm_w = static_cast<const bf16*>(q_norm_w);
  a.k_norm_w = static_cast<const bf16*>(k_norm_w);
  a.slot_mapping = slot_mapping;
  a.q_out = static_cast<bf16*>(q_out);
  a.k_out = static_cast<bf16*>(k_out);
  a.v_out = static_cast<bf16*>(v_out);
  a.k_cache = static_cast<bf16*>(k_cache);
  a.v_cache = static_cast<bf16*>(v_cache);
  a.num_slots = num_slots;
  return launch_tc<kTcQkvRope>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(w_qkv), n, a,
                               static_cast<cudaStream_t>(stream));
}

int64_t mdb_lmhead_workspace_bytes(int m, int vocab) {
  if (m <= 0 || vocab <= 0) return 0;
  return lmhead_layout(m, vocab).total;
}

int mdb_lmhead_sample(const void* hidden, int64_t ld_hidden, const void* w, int m, int vocab, int h,
                      const float* temperatures, int block, int noise_mode, const float* noise, uint32_t seed,
                      uint32_t step, const uint32_t* step_dev, void* workspace, int64_t workspace_bytes,
                      int32_t* x0_out, float* conf_out, mdb_stream_t stream) {
  MDB_REQUIRE(m >= 0 && vocab > 0 && h > 0 && block > 0, MDB_ERR_ARG);
  if (m == 0) return MDB_OK;
  MDB_REQUIRE(hidden && w && temperatures && x0_out && conf_out && workspace, MDB_ERR_ARG);
  MDB_REQUIRE(m % block == 0 && ld_hidden >= h, MDB_ERR_ARG);
  MDB_REQUIRE(noise_mode >= 0 && noise_mode <= 2 && (noise_mode != 1 || noise != nullptr), MDB_ERR_ARG);
  MDB_REQUIRE(ld_hidden % 8 == 0 && mdb_aligned16(hidden) && mdb_aligned16(w) && mdb_aligned16(workspace),
              MDB_ERR_ALIGN);
  const LmHeadLayout lay = lmhead_layout(m, vocab);
  MDB_REQUIRE(workspace_bytes >= lay.total, MDB_ERR_WORKSPACE);
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ws_supported(kWsLmHead, m, vocab, h, ld_hidden)) {
    WsArgs a = {};
    a.m = m; a.n = vocab; a.k = h; a.ksplit = 1;
    a.temperatures = temperatures;
    a.block = block;
    a.noise_mode = noise_mode;
    a.noise = noise;
    a.seed = seed; a.step = step;
    a.step_dev = step_dev;
    a.part_f = reinterpret_cast<float4*>(ws);
    a.part_i = reinterpret_cast<int*>(ws + lay.off_i);
    int rc = launch_ws<kWsLmHead>(static_cast<const bf16*>(hidden), ld_hidden, static_cast<const bf16*>(w), a, st);
    if (rc != MDB_OK) return rc;
    return finalize_sampler(a.part_f, a.part_i, vocab / kWsTileRows, m, x0_out, conf_out, st);
  }
  if (noise_mode != 1 && tc_supported(kTcLmHead, m, vocab, h, ld_hidden, 0)) {
    // tile GEMM whose epilogue reduces each 256-column tile to a sampler record
    TcArgs a = {};
    a.m = m; a.n = vocab; a.k = h;
    a.temperatures = temperatures;
    a.block = block;
    a.noise_mode = noise_mode;
    a.seed = seed; a.step = step;
    a.step_dev = step_dev;
    a.part_f = reinterpret_cast<float4*>(ws);
    a.part_i = reinterpret_cast<int*>(ws + lay.off_i);
    int rc = launch_tc<kTcLmHead>(static_cast<const bf16*>(hidden), ld_hidden, static_cast<const bf16*>(w), vocab, a, st);
    if (rc != MDB_OK) return rc;
    return finalize_sampler(a.part_f, a.part_i, a.tiles_n, m, x0_out, conf_out, st);
  }
  // an explicit noise tensor with many rows: bf16 logits in the workspace, then the scan
  MDB_REQUIRE(tc_supported(kTcBf16, m, vocab, h, ld_hidden, vocab), MDB_ERR_UNSUPPORTED);
  bf16* logits = reinterpret_cast<bf16*>(ws + lay.off_logits);
  TcArgs a = {};
  a.m = m; a.n = vocab; a.k = h;
  a.y = logits;
  a.ldy = vocab;
  int rc = launch_tc<kTcBf16>(static_cast<const bf16*>(hidden), ld_hidden, static_cast<const bf16*>(w), vocab, a, st);
  if (rc != MDB_OK) return rc;
  return scan_logits(logits, vocab, m, vocab, temperatures, block, noise_mode, noise, seed, step, step_dev, ws, x0_out,
                     conf_out, st);
}

int mdb_logits_sample(const void* logits, int64_t ld, int m, int vocab, const float* temperatures, int block,
                      int noise_mode, const float* noise, uint32_t seed, uint32_t step, const uint32_t* step_dev,
                      void* workspace, int64_t workspace_bytes, int32_t* x0_out, float* conf_out,
                      mdb_stream_t stream) {
  MDB_REQUIRE(m >= 0 && vocab > 0 && block > 0, MDB_ERR_ARG);
  if (m == 0) return MDB_OK;
  MDB_REQUIRE(logits && temperatures && x0_out && conf_out && workspace, MDB_ERR_ARG);
  MDB_REQUIRE(m % block == 0 && ld >= vocab, MDB_ERR_ARG);
  MDB_REQUIRE(noise_mode >= 0 && noise_mode <= 2 && (noise_mode != 1 || noise != nullptr), MDB_ERR_ARG);
  MDB_REQUIRE(mdb_aligned16(workspace), MDB_ERR_ALIGN);
  const int64_t nparts = (vocab + kScanCols - 1) / kScanCols;
  MDB_REQUIRE(workspace_bytes >= align256(nparts * m * 16) + align256(nparts * m * 4), MDB_ERR_WORKSPACE);
  return scan_logits(static_cast<const bf16*>(logits), ld, m, vocab, temperatures, block, noise_mode, noise, seed, step,
                     step_dev, static_cast<unsigned char*>(workspace), x0_out, conf_out, static_cast<cudaStream_t>(stream));
}

// ---- tensor-parallel pair (TP = 2) ----------------------------------------------------

int mdb_gemm_splitk_partials_tp(const void* x, int64_t ldx, const void* w, float* partials, float* peer_partials,
                                int m, int n, int k, int ksplit, uint32_t* peer_flags, uint32_t tag,
                                const uint32_t* epoch, mdb_stream_t stream) {
  if (m == 0) return MDB_OK;
  int rc = check_short_step(x, ldx, w, m, n, k);
  if (rc != MDB_OK) return rc;
  MDB_REQUIRE(partials && peer_partials && peer_flags && epoch && ksplit >= 1 && ksplit <= 64, MDB_ERR_ARG);
  MDB_REQUIRE(tag >= 1 && tag <= 255, MDB_ERR_ARG);
  MDB_REQUIRE(mdb_aligned16(partials) && mdb_aligned16(peer_partials), MDB_ERR_ALIGN);
  MDB_REQUIRE(ws_supported(kWsPartial, m, n, k, ldx), MDB_ERR_UNSUPPORTED);
  const int chunks = k / kWsBK;
  MDB_REQUIRE(((chunks + ksplit - 1) / ksplit) * (ksplit - 1) < chunks, MDB_ERR_ARG);
  WsArgs a = {};
  a.m = m; a.n = n; a.k = k; a.ksplit = ksplit;
  a.partials = partials;
  a.peer_partials = peer_partials;
  a.tp = TpSignal{peer_flags, nullptr, 0, tag, epoch};
  return launch_ws<kWsPartial>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(w), a,
                               static_cast<cudaStream_t>(stream));
}

int mdb_tp_grid_size(int m, int n, int k, int ksplit) {
  // CTAs (= flag slots) a streaming GEMM of this shape is launched with
  if (n % kWsTileRows != 0) return 0;
  const int tasks = n / kWsTileRows * (ksplit > 0 ? ksplit : 1);
  return tasks < 148 ? tasks : 148;
}

int mdb_lmhead_sample_tp(const void* hidden, int64_t ld_hidden, const void* w, int m, int vocab, int h,
                         const float* temperatures, int block, int noise_mode, const float* noise, uint32_t seed,
                         uint32_t step, const uint32_t* step_dev, void* workspace, void* peer_workspace,
                         int64_t workspace_bytes, int tile_begin, int tile_count, uint32_t* peer_flags,
                         const uint32_t* wait_flags, int wait_count, uint32_t tag, const uint32_t* epoch,
                         int32_t* x0_out, float* conf_out, mdb_stream_t stream) {
  MDB_REQUIRE(m >= 1 && vocab > 0 && h > 0 && block > 0, MDB_ERR_ARG);
  MDB_REQUIRE(hidden && w && temperatures && x0_out && conf_out && workspace && peer_workspace, MDB_ERR_ARG);
  MDB_REQUIRE(peer_flags && wait_flags && epoch && wait_count > 0 && tag >= 1 && tag <= 255, MDB_ERR_ARG);
  MDB_REQUIRE(m % block == 0 && ld_hidden >= h, MDB_ERR_ARG);
  MDB_REQUIRE(noise_mode >= 0 && noise_mode <= 2 && (noise_mode != 1 || noise != nullptr), MDB_ERR_ARG);
  if (m > 64) {
    // many rows: the tile GEMM over this rank's columns [128 tile_begin, 128 (tile_begin + tile_count)) of the
    // vocabulary, one record per 256-column tile; the shard must start on a 256-column boundary and end on one
    // or at the end of the vocabulary
    MDB_REQUIRE(noise_mode != 1 && vocab % 128 == 0, MDB_ERR_UNSUPPORTED);
    MDB_REQUIRE(tile_begin >= 0 && tile_count >= 1 && tile_begin % 2 == 0, MDB_ERR_ARG);
    const int64_t col_begin = static_cast<int64_t>(tile_begin) * 128;
    const int64_t col_end = col_begin + static_cast<int64_t>(tile_count) * 128;
    MDB_REQUIRE(col_end <= vocab && (col_end == vocab || col_end % kTcBN == 0), MDB_ERR_ARG);
    const int cols = static_cast<int>(col_end - col_begin);
    MDB_REQUIRE(tc_supported(kTcLmHead, m, cols, h, ld_hidden, 0), MDB_ERR_UNSUPPORTED);
    const LmHeadLayout lay = lmhead_layout(m, vocab);
    MDB_REQUIRE(workspace_bytes >= lay.off_logits, MDB_ERR_WORKSPACE);
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    unsigned char* pws = static_cast<unsigned char*>(peer_workspace);
    const int64_t rec0 = col_begin / kTcBN * m;            // first record of the shard
    TcArgs a = {};
    a.m = m; a.n = cols; a.k = h;
    a.temperatures = temperatures;
    a.block = block;
    a.noise_mode = noise_mode;
    a.seed = seed; a.step = step;
    a.step_dev = step_dev;
    a.part_f = reinterpret_cast<float4*>(ws) + rec0;
    a.part_i = reinterpret_cast<int*>(ws + lay.off_i) + rec0;
    a.peer_part_f = reinterpret_cast<float4*>(pws) + rec0;
    a.peer_part_i = reinterpret_cast<int*>(pws + lay.off_i) + rec0;
    a.col_base = static_cast<int>(col_begin);
    a.tp = TpSignal{peer_flags, nullptr, 0, tag, epoch};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bf16* w_shard = static_cast<const bf16*>(w) + col_begin * h;
    int rc = launch_tc_impl<kTcLmHead, false>(static_cast<const bf16*>(hidden), ld_hidden, w_shard, cols, a, st);
    if (rc != MDB_OK) return rc;
    const TpSignal wait = {nullptr, wait_flags, wait_count, tag, epoch};
    return finalize_sampler(reinterpret_cast<float4*>(ws), reinterpret_cast<int*>(ws + lay.off_i),
                            static_cast<int>(lay.nparts), m, x0_out, conf_out, st, wait);
  }
  MDB_REQUIRE(ws_supported(kWsLmHead, m, vocab, h, ld_hidden), MDB_ERR_UNSUPPORTED);
  const int tiles_total = vocab / kWsTileRows;
  MDB_REQUIRE(tile_begin >= 0 && tile_count >= 1 && tile_begin + tile_count <= tiles_total, MDB_ERR_ARG);
  const LmHeadLayout lay = lmhead_layout(m, vocab);
  MDB_REQUIRE(workspace_bytes >= lay.total, MDB_ERR_WORKSPACE);
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  unsigned char* pws = static_cast<unsigned char*>(peer_workspace);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  WsArgs a = {};
  a.m = m; a.n = vocab; a.k = h; a.ksplit = 1;
  a.temperatures = temperatures;
  a.block = block;
  a.noise_mode = noise_mode;
  a.noise = noise;
  a.seed = seed; a.step = step;
  a.step_dev = step_dev;
  a.part_f = reinterpret_cast<float4*>(ws);
  a.part_i = reinterpret_cast<int*>(ws + lay.off_i);
  a.peer_part_f = reinterpret_cast<float4*>(pws);
  a.peer_part_i = reinterpret_cast<int*>(pws + lay.off_i);
  a.tile_begin = tile_begin;
  a.tiles_override = tile_count;
  a.tp = TpSignal{peer_flags, nullptr, 0, tag, epoch};
  int rc = launch_ws<kWsLmHead>(static_cast<const bf16*>(hidden), ld_hidden, static_cast<const bf16*>(w), a, st);
  if (rc != MDB_OK) return rc;
  const TpSignal wait = {nullptr, wait_flags, wait_count, tag, epoch};
  return finalize_sampler(a.part_f, a.part_i, tiles_total, m, x0_out, conf_out, st, wait);
}

int64_t mdb_lmhead_tp_workspace_bytes(int m, int vocab) {
  if (m <= 0 || vocab <= 0) return 0;
  const LmHeadLayout lay = lmhead_layout(m, vocab);
  return m <= 64 ? lay.total : lay.off_logits;     // records only: the pair never materialises logits
}

int mdb_lmhead_tp_slots(int m, int cols) {
  if (m <= 64 || cols <= 0) return 0;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  const int64_t tiles = static_cast<int64_t>((m + kTcBM - 1) / kTcBM) * ((cols + kTcBN - 1) / kTcBN);
  return static_cast<int>(tiles < sms ? tiles : sms);
}

}  // extern "C"
