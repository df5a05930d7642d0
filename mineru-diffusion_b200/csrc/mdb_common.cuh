// Shared device/host helpers for the block-diffusion decode kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/mdb200.h"

namespace mdb {

typedef __nv_bfloat16 bf16;

constexpr int kHeadDim = 128;   // the only head size the SDAR decoder uses
constexpr int kPage = 256;      // tokens per KV page

// ---- device status word --------------------------------------------------
// Kernels never trap.  A soft check that fails (slot out of range, bounded
// wait expired) ORs a bit into this word and skips the access; the host reads
// it with mdb_last_device_status().
__device__ unsigned int g_device_status = 0;  // one definition: the library is a single translation unit

__device__ __forceinline__ void report_status(unsigned int bit) { atomicOr(&g_device_status, bit); }

// Longest time any wait inside a kernel (mbarrier, peer flag) may last before it gives up with
// MDB_STATUS_WAIT_TIMEOUT; 2 s unless MDB_OPT_WAIT_LIMIT_US says otherwise.  Read only on the slow path of a wait.
__device__ unsigned long long g_wait_limit_ns = 2000000000ull;

// ---- programmatic dependent launch ---------------------------------------------
// Every kernel of the library opens with pdl_launch_dependents() (the next
// kernel in the stream may be scheduled early, e.g. to prefetch weights) and
// calls pdl_wait() before it touches memory an earlier kernel may still write
// or read.  Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- optional device-side timeline (measurement aid) ---------------------------
// When a trace buffer is registered (mdb_set_trace), block 0 of the traced
// kernels appends (kernel id, event id, %globaltimer) triples to it.
struct TraceBuf {
  unsigned long long* data;   // [0] = count, then triples
  unsigned int capacity;      // triples
};
__device__ TraceBuf g_trace = {nullptr, 0};

__device__ __forceinline__ void trace_event(unsigned int kernel_id, unsigned int event_id) {
#ifndef MDB_TRACE
  // compiled out unless the library is built with -DMDB_TRACE: even the test of the buffer pointer is a global
  // load on the critical path of block 0 of every kernel
  (void)kernel_id;
  (void)event_id;
  return;
#endif
  if (blockIdx.x != 0 || blockIdx.y != 0 || blockIdx.z != 0) return;
  if (g_trace.data == nullptr) return;
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  const unsigned long long slot = atomicAdd(g_trace.data, 1ull);
  if (slot < g_trace.capacity) {
    g_trace.data[1 + 3 * slot] = kernel_id;
    g_trace.data[2 + 3 * slot] = event_id;
    g_trace.data[3 + 3 * slot] = t;
  }
}

// ---- tensor-parallel pair: signals over peer memory ------------------------------
// A producer kernel that has stored its partial results into the peer GPU's
// buffer publishes them by writing a sequence number into its CTA's slot of a
// flag array that also lives in the peer's memory (release at system scope).
// The consumer kernel on the peer waits, for a bounded time, until all slots
// carry that number.  The number is (step word in device memory) * 256 + tag,
// so it grows with every launch and a captured graph can be replayed.
struct TpSignal {
  unsigned int* peer_flags;        // producer side: slots in the peer's memory (one per CTA); null = no peer
  const unsigned int* wait_flags;  // consumer side: slots in local memory the peer writes; null = nothing to wait for
  int wait_count;
  unsigned int tag;                // 1..255, distinct per producing launch of a step
  const unsigned int* epoch;       // device word the host advances every step
};

__device__ __forceinline__ unsigned int tp_seq(const TpSignal& s) { return *s.epoch * 256u + s.tag; }

// Called by one thread of a CTA after the CTA's peer stores are complete (CTA-wide barrier before it).
__device__ __forceinline__ void tp_signal(const TpSignal& s) {
  if (s.peer_flags == nullptr) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(s.peer_flags + blockIdx.x), "r"(tp_seq(s)) : "memory");
}

// Called by every thread of a CTA; returns after all slots show the sequence number or the wait limit has passed
// (then MDB_STATUS_WAIT_TIMEOUT is raised and the kernel carries on with whatever the buffer holds).
__device__ __forceinline__ void tp_wait(const TpSignal& s) {
  if (s.wait_flags == nullptr) return;
  const unsigned int want = tp_seq(s);
  for (int i = threadIdx.x; i < s.wait_count; i += blockDim.x) {
    unsigned long long deadline = 0;
    for (unsigned int it = 0;; ++it) {
      unsigned int v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(s.wait_flags + i) : "memory");
      if (static_cast<int>(v - want) >= 0) break;
      if ((it & 255u) == 255u) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (deadline == 0) deadline = now + g_wait_limit_ns;
        else if (now > deadline) { report_status(MDB_STATUS_WAIT_TIMEOUT); break; }
      }
    }
  }
  __syncthreads();
}

// ---- small numeric helpers ------------------------------------------------
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Named barrier over `threads` threads that also ANDs a predicate across them.
__device__ __forceinline__ bool named_bar_and(int id, int threads, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, %2, %3, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(pred)), "r"(id), "r"(threads)
      : "memory");
  return r != 0;
}

// ---- counter-based Gumbel noise ---------------------------------------------
// One value per (seed, step, row, column); the LM-head scan and the noise dump
// entry point call the same function so a test can hand the exact noise to a
// CPU checker.
__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du;
  x ^= x >> 15; x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}

// The (seed, step, row) part of the hash, for callers that walk many columns of one row.
__device__ __forceinline__ uint32_t gumbel_row_key(uint32_t seed, uint32_t step, uint32_t row) {
  uint32_t h = mix32(seed ^ 0x9e3779b9u);
  h = mix32(h ^ (step * 0x85ebca6bu + 0xc2b2ae35u));
  return mix32(h ^ (row * 0x27d4eb2fu + 0x165667b1u));
}
__device__ __forceinline__ float gumbel_from_key(uint32_t row_key, uint32_t col) {
  const uint32_t h = mix32(row_key ^ col);
  // uniform in (0,1): 24 random bits, centred
  float u = (static_cast<float>(h >> 8) + 0.5f) * (1.0f / 16777216.0f);
  float e = -__logf(u);          // Exp(1)
  return -__logf(e);             // Gumbel(0,1), as -log(Exp(1)) in the reference sampler
}
__device__ __forceinline__ float gumbel_noise(uint32_t seed, uint32_t step, uint32_t row, uint32_t col) {
  return gumbel_from_key(gumbel_row_key(seed, step, row), col);
}

}  // namespace mdb

// ---- host-side argument checks ----------------------------------------------
#define MDB_REQUIRE(cond, code) \
  do {                          \
    if (!(cond)) return (code); \
  } while (0)

static inline bool mdb_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// process-wide options (mdb_set_option)
static int g_opt_pdl = 1;             // programmatic dependent launch between the library's kernels
static int g_opt_wait_limit_us = 2000000;   // bound of in-kernel waits (mirrors g_wait_limit_ns on the device)
static int g_opt_gemm_pair = 1;       // many-row GEMMs on CTA pairs (tcgen05.mma.cta_group::2): 1 from 2048 rows, 2 from 256, 0 never

// A kernel's opt-in attributes (dynamic shared memory above 48 KB) belong to one device's context, so the
// "already set" flag is kept per device ordinal: a process that drives several GPUs sets them on each.
struct PerDeviceOnce {
  bool done[64] = {};
  // Index of the current device's flag, or -1 when the device cannot be read or lies outside the table.
  int slot() const {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    return dev;
  }
};

// Launch with the programmatic-stream-serialization attribute when enabled.
template <typename... KArgs, typename... Args>
static inline int mdb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                             Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_opt_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...) == cudaSuccess ? MDB_OK : MDB_ERR_CUDA;
}

static inline int mdb_check_launch() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? MDB_OK : MDB_ERR_CUDA;
}
