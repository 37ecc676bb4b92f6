// A matrix per head: C[m, z, :] = W[z] · A[m, z, :] for every head z, bfloat16 on the tensor cores.
//
// The products around an attention over a cached latent are small per head (K and N are a head's
// size or the latent's rank, a few dozen to a few hundred) but there is one per head and token:
// as one launch, CTA (x, y, z) owns 64 rows x 64 columns of head z.  Both operands are staged in
// shared memory 64 k-columns at a time (16-byte loads where the addresses allow, guarded scalar
// loads at ragged edges), the four warps each own a 32 x 32 corner as 2 x 2 fragments of
// mma.sync (the warp-level matrix API), sums are 32-bit, and the tile leaves through shared
// memory so that its bfloat16 rows are written in 16-byte pieces.  Any M, N, K.
#include <mma.h>

#include "api.h"
#include "common.cuh"

namespace cretif {

namespace {
constexpr int kHM = 64, kHN = 64, kHK = 64, kHPad = 8;

__device__ __forceinline__ void stage_tile(__nv_bfloat16 (*dst)[kHK + kHPad],
                                           const __nv_bfloat16* __restrict__ src, int ld, int rows,
                                           int row0, int k0, int K, bool vec_ok) {
  // 64 rows x 64 columns, 8 columns (16 bytes) a thread and turn
  for (int idx = threadIdx.x; idx < kHM * (kHK / 8); idx += blockDim.x) {
    const int r = idx / (kHK / 8), c = (idx - r * (kHK / 8)) * 8;
    const int row = row0 + r, k = k0 + c;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < rows) {
      const __nv_bfloat16* p = src + (size_t)row * ld + k;
      if (vec_ok && k + 8 <= K) {
        v = *reinterpret_cast<const uint4*>(p);
      } else {
        __nv_bfloat16 tmp[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) tmp[e] = k + e < K ? p[e] : __float2bfloat16_rn(0.f);
        v = *reinterpret_cast<const uint4*>(tmp);
      }
    }
    *reinterpret_cast<uint4*>(&dst[r][c]) = v;
  }
}
}  // namespace

__global__ void __launch_bounds__(128)
gemm_heads_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                  __nv_bfloat16* __restrict__ C, int M, int N, int K, int lda, int ldc,
                  long long sa, long long sw, long long sc, int a_vec, int w_vec) {
  using namespace nvcuda;
  __shared__ __align__(32) __nv_bfloat16 As[kHM][kHK + kHPad];
  __shared__ __align__(32) __nv_bfloat16 Ws[kHN][kHK + kHPad];
  __shared__ __align__(32) float Cs[4][32][32 + 4];
  const int z = blockIdx.z;
  A += (size_t)z * sa;
  W += (size_t)z * sw;
  C += (size_t)z * sc;
  const int m0 = blockIdx.y * kHM, n0 = blockIdx.x * kHN;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[2][2];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) wmma::fill_fragment(acc[i][j], 0.f);
  for (int k0 = 0; k0 < K; k0 += kHK) {
    stage_tile(As, A, lda, M, m0, k0, K, a_vec);
    stage_tile(Ws, W, K, N, n0, k0, K, w_vec);
    __syncthreads();
    const int kk_end = min(kHK, ((K - k0 + 15) / 16) * 16);
    for (int kk = 0; kk < kk_end; kk += 16) {
      wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa[2];
      wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) wmma::load_matrix_sync(fa[i], &As[wm + 16 * i][kk], kHK + kHPad);
#pragma unroll
      for (int j = 0; j < 2; ++j) wmma::load_matrix_sync(fb[j], &Ws[wn + 16 * j][kk], kHK + kHPad);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) wmma::mma_sync(acc[i][j], fa[i], fb[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j)
      wmma::store_matrix_sync(&Cs[warp][16 * i][16 * j], acc[i][j], 32 + 4, wmma::mem_row_major);
  __syncwarp();
  // a lane writes row `lane` of its warp's corner
  const int row = m0 + wm + lane;
  if (row < M) {
    __nv_bfloat16* crow = C + (size_t)row * ldc + n0 + wn;
    const bool vec = ((reinterpret_cast<uintptr_t>(crow) & 15) == 0) && n0 + wn + 32 <= N;
    if (vec) {
#pragma unroll
      for (int c = 0; c < 32; c += 8) {
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = Cs[warp][lane][c + e];
        store8(crow + c, v);
      }
    } else {
      for (int c = 0; c < 32 && n0 + wn + c < N; ++c)
        crow[c] = __float2bfloat16_rn(Cs[warp][lane][c]);
    }
  }
}

}  // namespace cretif

using namespace cretif;

extern "C" int cretif_gemm_heads(const void* A, const void* W, void* C, int M, int N, int K,
                                 int lda, int ldc, int batch, long long sa, long long sc,
                                 void* stream) {
  if (M <= 0 || N <= 0 || batch <= 0) return kOk;
  if (K <= 0 || lda < K || ldc < N || batch > 65535 || (M + kHM - 1) / kHM > 65535)
    return kBadArgument;
  const int a_vec = ((uintptr_t)A % 16 == 0) && lda % 8 == 0 && sa % 8 == 0;
  const int w_vec = ((uintptr_t)W % 16 == 0) && K % 8 == 0;
  dim3 grid((N + kHN - 1) / kHN, (M + kHM - 1) / kHM, batch);
  gemm_heads_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, (__nv_bfloat16*)C, M, N, K, lda, ldc, sa,
      (long long)N * K, sc, a_vec, w_vec);
  return launch_status();
}
