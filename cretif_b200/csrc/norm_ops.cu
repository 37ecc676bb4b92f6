// Norms that sit elsewhere than in front of a sublayer.
//
// * rmsnorm_add: a norm on a sublayer's OUTPUT, fused with the residual addition:
//   h[t] += y[t] * w * rsqrt(mean(y[t]^2) + eps).  Sum, scaling and addition are 32-bit.
// * convert_rows: the residual stream handed to a sublayer that reads it without a norm
//   (float32 -> the compute type).
// * proj_norm_kv_append: RMS norms over whole query / key projections (all heads of a token
//   at once, one weight per channel), fused with the write into the block cache.  The key
//   part of a row is normed and stored as the key; when a value cache is given, the SAME
//   columns as projected (before the norm) are stored as the value: a layer whose values are
//   its keys needs no value projection.  Without query weights the query part is left alone,
//   without a value cache only keys are stored (a latent that serves as key and value).
#include "api.h"
#include "common.cuh"

namespace cretif {

template <typename TY>
__global__ void __launch_bounds__(256)
rmsnorm_add_kernel(float* __restrict__ h, const TY* __restrict__ y, int ldy,
                   const float* __restrict__ weight, int R, int H, float eps) {
  // a warp per row: no block-wide barrier, a row of up to 1024 columns stays in registers
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + warp;
  if (r >= R) return;
  const TY* yrow = y + (size_t)r * ldy;
  float* hrow = h + (size_t)r * H;
  constexpr int kKeep = 32;
  float keep[kKeep];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < kKeep; ++u) {
    const int i = u * 32 + lane;
    keep[u] = i < H ? to_float(yrow[i]) : 0.f;
    ss += keep[u] * keep[u];
  }
  for (int i = kKeep * 32 + lane; i < H; i += 32) {
    const float v = to_float(yrow[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int u = 0; u < kKeep; ++u) {
    const int i = u * 32 + lane;
    if (i < H) hrow[i] += keep[u] * inv * weight[i];
  }
  for (int i = kKeep * 32 + lane; i < H; i += 32)
    hrow[i] += to_float(yrow[i]) * inv * weight[i];
}

template <typename TO>
__global__ void convert_rows_kernel(const float* __restrict__ h, TO* __restrict__ out,
                                    size_t total) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) out[i] = from_float<TO>(h[i]);
}

template <typename T>
__global__ void __launch_bounds__(256)
proj_norm_kv_append_kernel(T* __restrict__ row0, int ld, int q_dim, const float* __restrict__ wq,
                           int nkv, int hd, const float* __restrict__ wk, float eps,
                           const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                           const int* __restrict__ seq_slot, const int* __restrict__ table,
                           int table_stride, T* __restrict__ kc, T* __restrict__ vc, int bt,
                           int write_cache, unsigned int* __restrict__ fault) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  T* row = row0 + (size_t)t * ld;
  const int kv_dim = nkv * hd;
  if (wq) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_dim; i += blockDim.x) {
      const float v = to_float(row[i]);
      ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)q_dim + eps);
    for (int i = threadIdx.x; i < q_dim; i += blockDim.x)
      row[i] = from_float<T>(to_float(row[i]) * inv * wq[i]);
  }
  T* krow = row + q_dim;
  float ss = 0.f;
  for (int i = threadIdx.x; i < kv_dim; i += blockDim.x) {
    const float v = to_float(krow[i]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  if (!write_cache) return;
  const float inv = 1.0f / sqrtf(ss / (float)kv_dim + eps);
  const int pos = tok_pos[t];
  const int slot = seq_slot[tok_seq[t]];
  const int blk = table[(size_t)slot * table_stride + pos / bt];
  if (blk < 0) {
    if (threadIdx.x == 0) atomicOr(fault, kFaultBlockTable);
    return;
  }
  const size_t cache_row = (size_t)blk * nkv * bt + (pos % bt);
  for (int i = threadIdx.x; i < kv_dim; i += blockDim.x) {
    const int kvh = i / hd, d = i - kvh * hd;
    const size_t at = (cache_row + (size_t)kvh * bt) * hd + d;
    const T raw = krow[i];
    kc[at] = from_float<T>(to_float(raw) * inv * wk[i]);
    if (vc) vc[at] = raw;
  }
}

}  // namespace cretif

using namespace cretif;

extern "C" int cretif_rmsnorm_add(float* h, const void* y, int y_dt, int ldy, const float* weight,
                                  int R, int H, float eps, void* stream) {
  if (R <= 0) return kOk;
  if (H <= 0 || ldy < H) return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((R + 7) / 8);
  if (y_dt == kF32)
    rmsnorm_add_kernel<float><<<blocks, 256, 0, st>>>(h, (const float*)y, ldy, weight, R, H, eps);
  else if (y_dt == kBF16)
    rmsnorm_add_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(h, (const __nv_bfloat16*)y, ldy,
                                                             weight, R, H, eps);
  else
    return kBadDType;
  return launch_status();
}

extern "C" int cretif_convert_rows(const float* h, void* out, int out_dt, long long total,
                                   void* stream) {
  if (total <= 0) return kOk;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (out_dt == kF32)
    convert_rows_kernel<float><<<blocks, 256, 0, st>>>(h, (float*)out, (size_t)total);
  else if (out_dt == kBF16)
    convert_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(h, (__nv_bfloat16*)out,
                                                              (size_t)total);
  else
    return kBadDType;
  return launch_status();
}

extern "C" int cretif_proj_norm_kv_append(void* rows, int ld, int dt, int q_dim, const float* wq,
                                          int nkv, int hd, const float* wk, float eps,
                                          const int* tok_pos, const int* tok_seq,
                                          const int* seq_slot, const int* table, int table_stride,
                                          void* kc, void* vc, int bt, int write_cache, int T,
                                          unsigned int* fault, void* stream) {
  if (T <= 0) return kOk;
  if (q_dim < 0 || nkv <= 0 || hd <= 0 || bt <= 0 || ld < q_dim + nkv * hd || !wk)
    return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
  if (dt == kF32)
    proj_norm_kv_append_kernel<float><<<T, 256, 0, st>>>(
        (float*)rows, ld, q_dim, wq, nkv, hd, wk, eps, tok_pos, tok_seq, seq_slot, table,
        table_stride, (float*)kc, (float*)vc, bt, write_cache, fault);
  else if (dt == kBF16)
    proj_norm_kv_append_kernel<__nv_bfloat16><<<T, 256, 0, st>>>(
        (__nv_bfloat16*)rows, ld, q_dim, wq, nkv, hd, wk, eps, tok_pos, tok_seq, seq_slot, table,
        table_stride, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, bt, write_cache, fault);
  else
    return kBadDType;
  return launch_status();
}
