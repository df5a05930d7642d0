// Peer memory for the tensor-parallel pair (TP = 2): buffers that the other
// GPU's kernels store into directly over NVLink (partial GEMM results, LM-head
// records, flag slots).  They are allocated once at engine start with
// cudaMalloc so that an IPC handle can be exported, exchanged through the
// process group by the host code, and opened by the peer process.  No kernel
// ever issues a TMA or multicast access to peer memory: only plain stores.
#include "mdb_common.cuh"

extern "C" {

int mdb_tp_alloc(int64_t bytes, void** out) {
  MDB_REQUIRE(bytes > 0 && out != nullptr, MDB_ERR_ARG);
  void* p = nullptr;
  if (cudaMalloc(&p, static_cast<size_t>(bytes)) != cudaSuccess) return MDB_ERR_CUDA;
  if (cudaMemset(p, 0, static_cast<size_t>(bytes)) != cudaSuccess) return MDB_ERR_CUDA;
  *out = p;
  return MDB_OK;
}

int mdb_tp_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? MDB_OK : MDB_ERR_CUDA; }

int mdb_tp_export(void* ptr, void* handle_out64) {
  MDB_REQUIRE(ptr && handle_out64, MDB_ERR_ARG);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) return MDB_ERR_CUDA;
  memcpy(handle_out64, &h, 64);
  return MDB_OK;
}

int mdb_tp_import(const void* handle64, void** peer_ptr_out) {
  MDB_REQUIRE(handle64 && peer_ptr_out, MDB_ERR_ARG);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return MDB_ERR_CUDA;
  *peer_ptr_out = p;
  return MDB_OK;
}

int mdb_tp_release(void* peer_ptr) { return cudaIpcCloseMemHandle(peer_ptr) == cudaSuccess ? MDB_OK : MDB_ERR_CUDA; }

}  // extern "C"
