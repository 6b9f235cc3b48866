// gemm_tcgen05.h - the tensor-core contraction of gemm_tcgen05.cu for callers that hold bf16 activations.
//
//   Y[M][N] (fp32) = residual + f(A[M][K] (bf16) . Wt[N][K]^T (bf16)),  fp32 accumulation in tensor memory
//
// f is the identity or a DynamicTanh per output column.  With row groups, the rows of A are sorted by group, every
// group starts on a multiple of kGemmRowTile rows, and group g multiplies rows [g * group_rows, g * group_rows + N)
// of Wt.
#pragma once

#include <cuda_runtime.h>

namespace dia {

constexpr int kGemmRowTile = 128;            // rows of A per output tile: the padding unit of a row group

struct GemmEpilogue {
    const float* residual;                   // [M][N] added to the result (may alias Y), or null
    const float* dyt_w;                      // [N]: f(a) = tanh(dyt_alpha a) dyt_w + dyt_b; null: f(a) = a
    const float* dyt_b;
    float dyt_alpha;
};

struct GemmGroups {
    const int* row_group;                    // device [M]: group of every row of A (read at the first row of a tile)
    int group_rows;                          // rows of Wt per group
    const int* n_rows;                       // device: rows of A in use (row tiles at or beyond it are skipped); null: M
};

// K a multiple of 8 (16-byte rows for the TMA), N a multiple of 4 (float4 stores)
inline bool gemm_tcgen05_shape_ok(int M, int N, int K) { return M > 0 && N > 0 && K >= 8 && K % 8 == 0 && N % 4 == 0; }

cudaError_t launch_gemm_tcgen05_bf16(const void* a_bf16, int terms, const void* wt, long long wt_rows, float* y, int M, int N,
                                     int K, const GemmEpilogue& ep, const GemmGroups* groups, cudaStream_t st);

}  // namespace dia
