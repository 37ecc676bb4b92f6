// Norms that sit elsewhere than in front of a sublayer.
//
// * rmsnorm_add: a norm on a sublayer's OUTPUT, fused with the residual addition:
//   h[t] += y[t] * w * rsqrt(mean(y[t]^2) + eps).  Sum, scaling and addition are 32-bit.  The
//   kernel can also leave the new rows in bfloat16 for the sublayer that reads them next.
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

namespace {
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                     __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
}
__device__ __forceinline__ void st4_bf16(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}
}  // namespace

// A warp per row, no block-wide barrier.  VEC: rows are read and written four columns at a time
// (H and the row strides multiples of 4, 16-byte aligned bases) and a row of up to 2048 columns
// stays in registers between the sum of squares and the addition; every loop is unrolled so
// that a lane's loads are in flight together (a step of one token is one warp, and a loop that
// waited for each load in turn took longer than the product before it).
template <typename TY, bool VEC>
__global__ void __launch_bounds__(256)
rmsnorm_add_kernel(float* __restrict__ h, const TY* __restrict__ y, int ldy,
                   const float* __restrict__ weight, int R, int H, float eps,
                   __nv_bfloat16* __restrict__ x_out) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + warp;
  if (r >= R) return;
  const TY* yrow = y + (size_t)r * ldy;
  float* hrow = h + (size_t)r * H;
  __nv_bfloat16* xrow = x_out ? x_out + (size_t)r * H : nullptr;
  if (VEC) {
    constexpr int kKeep = 16;
    const int n4 = H >> 2;
    float4 keep[kKeep];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < kKeep; ++u) {
      const int i = u * 32 + lane;
      keep[u] = i < n4 ? ld4(yrow + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
      ss += keep[u].x * keep[u].x + keep[u].y * keep[u].y + keep[u].z * keep[u].z +
            keep[u].w * keep[u].w;
    }
#pragma unroll 4
    for (int i = kKeep * 32 + lane; i < n4; i += 32) {
      const float4 v = ld4(yrow + 4 * i);
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int u = 0; u < kKeep; ++u) {
      const int i = u * 32 + lane;
      if (i < n4) {
        const float4 w = ld4(weight + 4 * i);
        float4 v = ld4(hrow + 4 * i);
        v.x += keep[u].x * inv * w.x; v.y += keep[u].y * inv * w.y;
        v.z += keep[u].z * inv * w.z; v.w += keep[u].w * inv * w.w;
        *reinterpret_cast<float4*>(hrow + 4 * i) = v;
        if (xrow) st4_bf16(xrow + 4 * i, v);
      }
    }
#pragma unroll 4
    for (int i = kKeep * 32 + lane; i < n4; i += 32) {
      const float4 w = ld4(weight + 4 * i), a = ld4(yrow + 4 * i);
      float4 v = ld4(hrow + 4 * i);
      v.x += a.x * inv * w.x; v.y += a.y * inv * w.y; v.z += a.z * inv * w.z; v.w += a.w * inv * w.w;
      *reinterpret_cast<float4*>(hrow + 4 * i) = v;
      if (xrow) st4_bf16(xrow + 4 * i, v);
    }
    return;
  }
  float ss = 0.f;
#pragma unroll 8
  for (int i = lane; i < H; i += 32) {
    const float v = to_float(yrow[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll 8
  for (int i = lane; i < H; i += 32) {
    const float v = hrow[i] + to_float(yrow[i]) * inv * weight[i];
    hrow[i] = v;
    if (xrow) xrow[i] = __float2bfloat16_rn(v);
  }
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
#pragma unroll 4
    for (int i = threadIdx.x; i < q_dim; i += blockDim.x) {
      const float v = to_float(row[i]);
      ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)q_dim + eps);
#pragma unroll 4
    for (int i = threadIdx.x; i < q_dim; i += blockDim.x)
      row[i] = from_float<T>(to_float(row[i]) * inv * wq[i]);
  }
  T* krow = row + q_dim;
  float ss = 0.f;
#pragma unroll 4
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
#pragma unroll 4
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
                                  int R, int H, float eps, void* x_out, void* stream) {
  if (R <= 0) return kOk;
  if (H <= 0 || ldy < H) return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((R + 7) / 8);
  const bool vec = H % 4 == 0 && ldy % 4 == 0 &&
                   (((uintptr_t)h | (uintptr_t)y | (uintptr_t)weight | (uintptr_t)x_out) & 15) == 0;
  __nv_bfloat16* xo = (__nv_bfloat16*)x_out;
  if (y_dt == kF32) {
    if (vec) rmsnorm_add_kernel<float, true><<<blocks, 256, 0, st>>>(h, (const float*)y, ldy, weight, R, H, eps, xo);
    else rmsnorm_add_kernel<float, false><<<blocks, 256, 0, st>>>(h, (const float*)y, ldy, weight, R, H, eps, xo);
  } else if (y_dt == kBF16) {
    typedef __nv_bfloat16 bf16;
    if (vec) rmsnorm_add_kernel<bf16, true><<<blocks, 256, 0, st>>>(h, (const bf16*)y, ldy, weight, R, H, eps, xo);
    else rmsnorm_add_kernel<bf16, false><<<blocks, 256, 0, st>>>(h, (const bf16*)y, ldy, weight, R, H, eps, xo);
  } else {
    return kBadDType;
  }
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
