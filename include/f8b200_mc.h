/*
 * f8b200_mc.h -- C ABI of libf8b200_mc.so, the optional cluster-multicast variant of the scaled
 * fp8 GEMM of f8b200.h (same reference call site: addmm_float8_unwrapped -> torch._scaled_mm,
 * float8_experimental/float8_python_api.py:24-64).
 *
 * FOR JOBS THAT USE ONE GPU ONLY.  Its kernels fetch operand tiles with TMA loads that multicast
 * to the CTAs of a thread-block cluster.  Such a load must never read another GPU's memory, so
 *   - the library is not shipped to, built for or loaded by runs on two or more GPUs;
 *   - the entry point itself refuses (F8B200_ERR_UNSUPPORTED, nothing launched) any operand or
 *     output pointer that is not ordinary device memory owned by the CURRENT device (peer
 *     pointers, IPC / symmetric-memory mappings, managed and host memory are all refused).
 * Callers fall back to f8b200_gemm_fp8_ws on F8B200_ERR_UNSUPPORTED.
 */
#ifndef F8B200_MC_H_
#define F8B200_MC_H_

#include "f8b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/*
 * f8b200_gemm_fp8_ws computed by clusters of cluster_m x cluster_n CTAs (2x1 or 2x2: one 256x256
 * tile per CTA, the CTAs of a cluster row share A and those of a column share B; 4x1: two
 * cta_group::2 pairs sharing B, K-major operands only).  `workspace` may be NULL (fixed tile
 * stride).  Results are bit-identical to f8b200_gemm_fp8.
 */
int f8b200_mc_gemm_fp8(const void* a, int a_kind, int a_layout, int64_t lda, const void* b, int b_kind,
                       int b_layout, int64_t ldb, const float* scale_a, const float* scale_b,
                       const void* bias, int out_dtype, void* out, int64_t ldo, int64_t m, int64_t n,
                       int64_t k, int cluster_m, int cluster_n, void* workspace, int64_t workspace_bytes,
                       void* stream);

/* f8b200_read_device_error for the error word of this library's own kernels. */
int f8b200_mc_read_device_error(uint32_t* flags_out);

#ifdef __cplusplus
}
#endif
#endif /* F8B200_MC_H_ */
