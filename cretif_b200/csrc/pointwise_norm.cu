// Dynamic Tanh, a norm without statistics, and the token shift that can follow it.
//
//     dyt(x)[c] = (tanh(alpha * x[c]) * w[c] + b[c]) * gain[c]        (gain optional)
//
// Every element is on its own, so the kernels are a thread per VEC columns -- four where the
// width and every address allow 16-byte accesses, else one -- and all arithmetic is 32-bit
// (tanhf).
//
// * dyt_rows: v = h[src] (+ delta[src]); if write_h, h[src] = v; out[r] = dyt(v), in float32 or
//   bfloat16.  src = rows ? rows[r] : r.
// * dyt_add: h[r] += dyt(y[r]) -- the norm on a sublayer's OUTPUT, fused with the residual sum.
// * shift_rows: a row blended with the row of the token before it,
//       out[t] = n[t] + (n[t-1] - n[t]) * shift,      n[t] = dyt(h[t])  (or h[t] without a norm)
//   where the first token of a sequence's portion takes n[t-1] from the sequence's saved row
//   (zeros at a sequence's start: a slot's state is zeroed when it is handed out).  The thread
//   that reads the saved row then replaces it by the portion's last row, so that no other thread
//   reads what it overwrites; a sequence of one token reads and writes in one thread.
#include "api.h"
#include "common.cuh"

namespace cretif {

namespace {

struct DytParams {
  const float* w;        // null: the identity (no norm)
  const float* b;
  const float* alpha;    // one number on the device
  const float* gain;     // may be null
};

__device__ __forceinline__ float4 ld4v(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4v(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                     __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
}
__device__ __forceinline__ void st4v(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4v(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}

__device__ __forceinline__ float dyt1(float v, float alpha, const DytParams& p, int c) {
  if (!p.w) return v;
  float r = tanhf(alpha * v) * p.w[c] + p.b[c];
  if (p.gain) r *= p.gain[c];
  return r;
}

template <int VEC> struct Pack { float v[VEC]; };

template <int VEC, typename T>
__device__ __forceinline__ Pack<VEC> ld_pack(const T* p) {
  Pack<VEC> r;
  if constexpr (VEC == 4) {
    const float4 f = ld4v(p);
    r.v[0] = f.x; r.v[1] = f.y; r.v[2] = f.z; r.v[3] = f.w;
  } else {
    r.v[0] = to_float(p[0]);
  }
  return r;
}

template <int VEC, typename T>
__device__ __forceinline__ void st_pack(T* p, const Pack<VEC>& r) {
  if constexpr (VEC == 4) st4v(p, make_float4(r.v[0], r.v[1], r.v[2], r.v[3]));
  else p[0] = from_float<T>(r.v[0]);
}

template <int VEC>
__device__ __forceinline__ Pack<VEC> dyt_pack(const Pack<VEC>& x, float alpha, const DytParams& p,
                                              int c) {
  Pack<VEC> r;
#pragma unroll
  for (int i = 0; i < VEC; ++i) r.v[i] = dyt1(x.v[i], alpha, p, c + i);
  return r;
}

template <typename TD, typename TO, int VEC>
__global__ void __launch_bounds__(256)
dyt_rows_kernel(float* __restrict__ h, const TD* __restrict__ delta, DytParams p,
                TO* __restrict__ out, const int* __restrict__ rows, int R, int H, int write_h) {
  const long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (idx >= (long long)R * H) return;
  const int r = (int)(idx / H), c = (int)(idx - (long long)r * H);
  const int src = rows ? rows[r] : r;
  Pack<VEC> v = ld_pack<VEC>(h + (size_t)src * H + c);
  if (delta) {
    const Pack<VEC> dl = ld_pack<VEC>(delta + (size_t)src * H + c);
#pragma unroll
    for (int i = 0; i < VEC; ++i) v.v[i] += dl.v[i];
    if (write_h) st_pack<VEC>(h + (size_t)src * H + c, v);
  }
  st_pack<VEC>(out + (size_t)r * H + c, dyt_pack<VEC>(v, p.alpha ? *p.alpha : 1.f, p, c));
}

template <typename TY, int VEC>
__global__ void __launch_bounds__(256)
dyt_add_kernel(float* __restrict__ h, const TY* __restrict__ y, int ldy, DytParams p, int R,
               int H) {
  const long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (idx >= (long long)R * H) return;
  const int r = (int)(idx / H), c = (int)(idx - (long long)r * H);
  const Pack<VEC> n = dyt_pack<VEC>(ld_pack<VEC>(y + (size_t)r * ldy + c),
                                    p.alpha ? *p.alpha : 1.f, p, c);
  Pack<VEC> v = ld_pack<VEC>(h + (size_t)r * H + c);
#pragma unroll
  for (int i = 0; i < VEC; ++i) v.v[i] += n.v[i];
  st_pack<VEC>(h + (size_t)r * H + c, v);
}

template <typename TO, int VEC>
__global__ void __launch_bounds__(256)
shift_rows_kernel(const float* __restrict__ h, DytParams p, const float* __restrict__ shift,
                  float* __restrict__ state, size_t state_stride,
                  const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                  const int* __restrict__ cu_seqlens, TO* __restrict__ out, int T, int H) {
  const long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (idx >= (long long)T * H) return;
  const int t = (int)(idx / H), c = (int)(idx - (long long)t * H);
  const float alpha = p.alpha ? *p.alpha : 1.f;
  const int b = tok_seq[t];
  const int first = cu_seqlens[b];
  const Pack<VEC> n = dyt_pack<VEC>(ld_pack<VEC>(h + (size_t)t * H + c), alpha, p, c);
  Pack<VEC> prev;
  if (t == first) {
    float* s = state + (size_t)seq_slot[b] * state_stride + c;
    prev = ld_pack<VEC>(s);
    const int last = cu_seqlens[b + 1] - 1;
    st_pack<VEC>(s, last == t ? n : dyt_pack<VEC>(ld_pack<VEC>(h + (size_t)last * H + c), alpha,
                                                   p, c));
  } else {
    prev = dyt_pack<VEC>(ld_pack<VEC>(h + (size_t)(t - 1) * H + c), alpha, p, c);
  }
  const Pack<VEC> sh = ld_pack<VEC>(shift + c);
  Pack<VEC> o;
#pragma unroll
  for (int i = 0; i < VEC; ++i) o.v[i] = n.v[i] + (prev.v[i] - n.v[i]) * sh.v[i];
  st_pack<VEC>(out + (size_t)t * H + c, o);
}

inline unsigned blocks_for(long long n) { return (unsigned)((n + 255) / 256); }

template <typename... P>
inline bool aligned16(const P*... ptrs) {
  return ((... | (uintptr_t)ptrs) & 15) == 0;
}

}  // namespace
}  // namespace cretif

using namespace cretif;

extern "C" int cretif_dyt_rows(float* h, const void* delta, int delta_dt, const float* w,
                               const float* b, const float* alpha, const float* gain, void* out,
                               int out_dt, const int* rows, int R, int H, int write_h,
                               void* stream) {
  if (R <= 0) return kOk;
  if (H <= 0 || !w || !b || !alpha || (rows && write_h)) return kBadArgument;
  if ((long long)R * H > 0x7fffffffLL * 256) return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
  const DytParams p{w, b, alpha, gain};
  const bool vec = H % 4 == 0 && aligned16(h, delta, w, b, gain, out);
  const unsigned g = blocks_for(((long long)R * H + (vec ? 3 : 0)) / (vec ? 4 : 1));
  typedef __nv_bfloat16 bf16;
  if (delta && delta_dt != kF32 && delta_dt != kBF16) return kBadDType;
#define CRETIF_DYT(TD, TO)                                                                      \
  do {                                                                                          \
    if (vec) dyt_rows_kernel<TD, TO, 4><<<g, 256, 0, st>>>(h, (const TD*)delta, p, (TO*)out,     \
                                                           rows, R, H, write_h);                 \
    else dyt_rows_kernel<TD, TO, 1><<<g, 256, 0, st>>>(h, (const TD*)delta, p, (TO*)out, rows,  \
                                                       R, H, write_h);                           \
  } while (0)
  const bool dbf = delta && delta_dt == kBF16;
  if (out_dt == kF32) {
    if (dbf) CRETIF_DYT(bf16, float); else CRETIF_DYT(float, float);
  } else if (out_dt == kBF16) {
    if (dbf) CRETIF_DYT(bf16, bf16); else CRETIF_DYT(float, bf16);
  } else {
    return kBadDType;
  }
#undef CRETIF_DYT
  return launch_status();
}

extern "C" int cretif_dyt_add(float* h, const void* y, int y_dt, int ldy, const float* w,
                              const float* b, const float* alpha, const float* gain, int R, int H,
                              void* stream) {
  if (R <= 0) return kOk;
  if (H <= 0 || ldy < H || !w || !b || !alpha) return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
  const DytParams p{w, b, alpha, gain};
  const bool vec = H % 4 == 0 && ldy % 4 == 0 && aligned16(h, y, w, b, gain);
  const unsigned g = blocks_for(((long long)R * H + (vec ? 3 : 0)) / (vec ? 4 : 1));
  typedef __nv_bfloat16 bf16;
  if (y_dt == kF32) {
    if (vec) dyt_add_kernel<float, 4><<<g, 256, 0, st>>>(h, (const float*)y, ldy, p, R, H);
    else dyt_add_kernel<float, 1><<<g, 256, 0, st>>>(h, (const float*)y, ldy, p, R, H);
  } else if (y_dt == kBF16) {
    if (vec) dyt_add_kernel<bf16, 4><<<g, 256, 0, st>>>(h, (const bf16*)y, ldy, p, R, H);
    else dyt_add_kernel<bf16, 1><<<g, 256, 0, st>>>(h, (const bf16*)y, ldy, p, R, H);
  } else {
    return kBadDType;
  }
  return launch_status();
}

extern "C" int cretif_shift_rows(const float* h, const float* w, const float* b,
                                 const float* alpha, const float* shift, float* state,
                                 long long state_stride, const int* tok_seq, const int* seq_slot,
                                 const int* cu_seqlens, void* out, int out_dt, int T, int H,
                                 void* stream) {
  if (T <= 0) return kOk;
  if (H <= 0 || !shift || !state || state_stride < H || (w && (!b || !alpha))) return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
  const DytParams p{w, b, alpha, nullptr};
  const bool vec = H % 4 == 0 && state_stride % 4 == 0 && aligned16(h, w, b, shift, state, out);
  const unsigned g = blocks_for(((long long)T * H + (vec ? 3 : 0)) / (vec ? 4 : 1));
  typedef __nv_bfloat16 bf16;
#define CRETIF_SHIFT(TO, V)                                                                     \
  shift_rows_kernel<TO, V><<<g, 256, 0, st>>>(h, p, shift, state, (size_t)state_stride, tok_seq, \
                                              seq_slot, cu_seqlens, (TO*)out, T, H)
  if (out_dt == kF32) {
    if (vec) CRETIF_SHIFT(float, 4); else CRETIF_SHIFT(float, 1);
  } else if (out_dt == kBF16) {
    if (vec) CRETIF_SHIFT(bf16, 4); else CRETIF_SHIFT(bf16, 1);
  } else {
    return kBadDType;
  }
#undef CRETIF_SHIFT
  return launch_status();
}
