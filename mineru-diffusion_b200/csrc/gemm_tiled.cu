// y = x W^T for many rows (prefill, large decode batches): a shared-memory
// tiled tensor-core GEMM.  CTA tile 128 x 128 x 64, 8 warps (2 x 4, warp tile
// 64 x 32), 3-stage cp.async ring, XOR-swizzled 128-byte rows read with
// ldmatrix, fp32 accumulation, one rounding to bf16 at the store.  Both
// operands are k-contiguous ("TN").
#include "mdb_common.cuh"

namespace mdb {

constexpr int kGemmBM = 128, kGemmBN = 128, kGemmBK = 64;
constexpr int kGemmStages = 3;
constexpr int kGemmThreads = 256;
constexpr int kGemmTileBytes = kGemmBM * kGemmBK * 2;                   // 16 KB per operand per stage
constexpr int kGemmSmemBytes = kGemmStages * 2 * kGemmTileBytes;        // 96 KB

__global__ void __launch_bounds__(kGemmThreads)
gemm_tiled_kernel(const bf16* __restrict__ x, int64_t ldx, const bf16* __restrict__ w, bf16* __restrict__ y,
                  int64_t ldy, int m, int n, int k) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const uint32_t smem = smem_u32(smem_raw);
  const int m0 = blockIdx.y * kGemmBM, n0 = blockIdx.x * kGemmBN;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = warp >> 2, wn = warp & 3;  // warp tile origin: rows 64*wm, cols 32*wn
  const int g = lane >> 2, t = lane & 3;
  const int mat = lane >> 3, r8 = lane & 7;
  const int ktiles = k / kGemmBK;

  auto issue = [&](int kt, int stage) {
    const uint32_t at = smem + stage * 2 * kGemmTileBytes;
    const uint32_t bt = at + kGemmTileBytes;
    const int chunk = threadIdx.x & 7;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = (threadIdx.x >> 3) + 32 * i;
      const uint32_t off = row * 128 + (swz_chunk(row, chunk) << 4);
      const bool av = m0 + row < m;
      const bool bv = n0 + row < n;
      const bf16* asrc = x + static_cast<int64_t>(av ? m0 + row : 0) * ldx + kt * kGemmBK + chunk * 8;
      const bf16* bsrc = w + static_cast<int64_t>(bv ? n0 + row : 0) * k + kt * kGemmBK + chunk * 8;
      cp_async16(at + off, asrc, av ? 16 : 0);
      cp_async16(bt + off, bsrc, bv ? 16 : 0);
    }
  };

  float acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

#pragma unroll
  for (int s = 0; s < kGemmStages - 1; ++s) {
    if (s < ktiles) issue(s, s);
    cp_async_commit();
  }
  for (int kt = 0; kt < ktiles; ++kt) {
    cp_async_wait<kGemmStages - 2>();
    __syncthreads();
    const int nxt = kt + kGemmStages - 1;
    if (nxt < ktiles) issue(nxt, nxt % kGemmStages);
    cp_async_commit();

    const uint32_t at = smem + (kt % kGemmStages) * 2 * kGemmTileBytes;
    const uint32_t bt = at + kGemmTileBytes;
#pragma unroll
    for (int ks = 0; ks < kGemmBK / 16; ++ks) {
      uint32_t af[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = 64 * wm + 16 * i + (mat & 1) * 8 + r8;
        const int chunk = 2 * ks + (mat >> 1);
        ldmatrix_x4(af[i][0], af[i][1], af[i][2], af[i][3], at + row * 128 + (swz_chunk(row, chunk) << 4));
      }
#pragma unroll
      for (int jp = 0; jp < 2; ++jp) {
        const int row = 32 * wn + 16 * jp + (mat >> 1) * 8 + r8;
        const int chunk = 2 * ks + (mat & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, bt + row * 128 + (swz_chunk(row, chunk) << 4));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          mma_bf16_16816(acc[i][2 * jp], af[i][0], af[i][1], af[i][2], af[i][3], b0, b1);
          mma_bf16_16816(acc[i][2 * jp + 1], af[i][0], af[i][1], af[i][2], af[i][3], b2, b3);
        }
      }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r0 = m0 + 64 * wm + 16 * i + g, r1 = r0 + 8;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + 32 * wn + 8 * j + 2 * t;
      if (c < n) {
        if (r0 < m) *reinterpret_cast<uint32_t*>(y + r0 * ldy + c) = pack_bf16x2(acc[i][j][0], acc[i][j][1]);
        if (r1 < m) *reinterpret_cast<uint32_t*>(y + r1 * ldy + c) = pack_bf16x2(acc[i][j][2], acc[i][j][3]);
      }
    }
  }
}

int launch_gemm_tiled(const bf16* x, int64_t ldx, const bf16* w, bf16* y, int64_t ldy, int m, int n, int k,
                      cudaStream_t st) {
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes) !=
        cudaSuccess)
      return MDB_ERR_CUDA;
    attr_set = true;
  }
  dim3 grid((n + kGemmBN - 1) / kGemmBN, (m + kGemmBM - 1) / kGemmBM);
  return mdb_launch(gemm_tiled_kernel, grid, dim3(kGemmThreads), kGemmSmemBytes, st, x, ldx, w, y, ldy, m, n, k);
}

}  // namespace mdb
