// Build wrapper for the reference's own device code (test infrastructure only).
//
// The reference assembles one NVRTC translation unit from its .cu fragments in the order
// given by crates/core/src/cuda/kernels/mod.rs:8-18.  This file reproduces that order with
// #include directives that resolve against the reference checkout through -I, so that no
// reference source is copied.  oracle/Makefile compiles it to oracle/_ref/ref_kernels.cubin
// with the reference's compile options (crates/core/src/cuda/device.rs:106-120: ftz, no
// precise div/sqrt, fmad, fast math) for sm_100, the target its NVRTC call picks on a B200.
#include "kernels/common.cu"
#include "kernels/gemm.cu"
#include "kernels/gemv.cu"
#include "kernels/embed.cu"
#include "kernels/ops.cu"
#include "kernels/deltanet.cu"
#include "kernels/attn/fast_v2.cu"
#include "kernels/attn/flash.cu"
