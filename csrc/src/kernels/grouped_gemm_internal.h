// Internal interface between the two grouped-GEMM kernels and their common launcher.
#ifndef NIXL_B200_GROUPED_GEMM_INTERNAL_H
#define NIXL_B200_GROUPED_GEMM_INTERNAL_H

#include <cuda.h>
#include <cuda_runtime.h>

#include "kernels/nixl_kernels.h"

namespace nixl_gemm {

enum : int { GEMM_ERR_TIMEOUT = 1, GEMM_ERR_ARRIVAL = 2 };
constexpr int kMaxGroups = 512;

// 2-D tensor map over a row-major [rows, k] byte matrix, boxes of box_rows x 128 bytes, 128-byte swizzle.
bool makeTileMap(CUtensorMap *map, const void *base, uint64_t rows, uint64_t k, uint32_t box_rows = 128);

// 256 x 256 tiles computed by CTA pairs (tcgen05 cta_group::2).  Same contract as the
// single-CTA kernel; N must be a multiple of 256.
cudaError_t launchPairKernel(const CUtensorMap &mapA, const CUtensorMap &mapW, const NixlGroupedGemmParams &p, cudaStream_t stream);

// Same tiles with power-of-two block scales applied by the tensor core (kind::mxf8f6f4.block_scale):
// p.scale_a / p.scale_w point at exponent bytes (uint8 [a_rows][K/128] and [groups][N/128][K/128]);
// K must be a multiple of 512, N of 256; no dispatch overlap.
cudaError_t launchMxPairKernel(const CUtensorMap &mapA, const CUtensorMap &mapW, const NixlGroupedGemmParams &p, cudaStream_t stream);

} // namespace nixl_gemm

#endif
