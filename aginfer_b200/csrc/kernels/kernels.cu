// The sm_100a kernel bundle of the AIM artifact set: one translation unit -> one CUBIN.
//   nvcc -cubin -arch=sm_100a -O3 -o kernels.cubin kernels.cu
#include "elementwise.cuh"
#include "norm.cuh"
#include "rope.cuh"
#include "vision.cuh"
#include "attention.cuh"
#include "attention_fa.cuh"
#include "gemm_simt.cuh"
#include "gemm_tc.cuh"
#include "gemm_tc_wide.cuh"
#include "gemm_tc_persist.cuh"
#include "gemm_skinny.cuh"
#include "gemm_stream.cuh"
