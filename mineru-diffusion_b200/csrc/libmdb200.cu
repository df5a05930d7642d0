// Single translation unit of libmdb200.so: the kernels share one device status
// word and a few launch helpers, so the parts are included here in order
// rather than linked as relocatable device code.
#include "elementwise.cu"
#include "attention.cu"
#include "sampler.cu"
#include "gemm_ws.cu"
#include "gemm_tc.cu"
#include "attention_tc.cu"
#include "api_linear.cu"
#include "tp_p2p.cu"
