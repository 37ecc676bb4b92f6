// Dynamic Tanh, a norm without statistics, and the token shift that can follow it.
//
//     dyt(x)[c] = (tanh(alpha * x[c]) * w[c] + b[c]) * gain[c]        (gain optional)
//
// Every element is on its own, so the kernels are a thread per four columns (per column where
// the width or an address is not a multiple of four) and all arithmetic is 32-bit (tanhf).
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

__device__ __forceinline__ float dyt1(float v, float alpha, const DytParams& p, int c) {
  if (!p.w) return v;
  float r = tanhf(alpha * v) * p.w[c] + p.b[c];
  if (p.gain) r *= p.gain[c];
  return r;
}

template <typename TD, typename TO>
__global__ void __launch_bounds__(256)
dyt_rows_kernel(float* __restrict__ h, const TD* __restrict__ delta, DytParams p,
                TO* __restrict__ out, const int* __restrict__ rows, int R, int H, int write_h) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)R * H) return;
  const int r = (int)(idx / H), c = (int)(idx - (long long)r * H);
  const int src = rows ? rows[r] : r;
  float v = h[(size_t)src * H + c];
  if (delta) {
    v += to_float(delta[(size_t)src * H + c]);
    if (write_h) h[(size_t)src * H + c] = v;
  }
  out[(size_t)r * H + c] = from_float<TO>(dyt1(v, p.alpha ? *p.alpha : 1.f, p, c));
}

template <typename TY>
__global__ void __launch_bounds__(256)
dyt_add_kernel(float* __restrict__ h, const TY* __restrict__ y, int ldy, DytParams p, int R,
               int H) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)R * H) return;
  const int r = (int)(idx / H), c = (int)(idx - (long long)r * H);
  const float v = to_float(y[(size_t)r * ldy + c]);
  h[(size_t)r * H + c] += dyt1(v, p.alpha ? *p.alpha : 1.f, p, c);
}

template <typename TO>
__global__ void __launch_bounds__(256)
shift_rows_kernel(const float* __restrict__ h, DytParams p, const float* __restrict__ shift,
                  float* __restrict__ state, size_t state_stride,
                  const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                  const int* __restrict__ cu_seqlens, TO* __restrict__ out, int T, int H) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * H) return;
  const int t = (int)(idx / H), c = (int)(idx - (long long)t * H);
  const float alpha = p.alpha ? *p.alpha : 1.f;
  const int b = tok_seq[t];
  const int first = cu_seqlens[b];
  const float n = dyt1(h[(size_t)t * H + c], alpha, p, c);
  float prev;
  if (t == first) {
    float* s = state + (size_t)seq_slot[b] * state_stride + c;
    prev = *s;
    const int last = cu_seqlens[b + 1] - 1;
    *s = last == t ? n : dyt1(h[(size_t)last * H + c], alpha, p, c);
  } else {
    prev = dyt1(h[(size_t)(t - 1) * H + c], alpha, p, c);
  }
  out[(size_t)t * H + c] = from_float<TO>(n + (prev - n) * shift[c]);
}

inline unsigned blocks_for(long long n) { return (unsigned)((n + 255) / 256); }

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
  const unsigned g = blocks_for((long long)R * H);
  typedef __nv_bfloat16 bf16;
  if (delta && delta_dt != kF32 && delta_dt != kBF16) return kBadDType;
#define CRETIF_DYT(TD, TO)                                                                      \
  dyt_rows_kernel<TD, TO><<<g, 256, 0, st>>>(h, (const TD*)delta, p, (TO*)out, rows, R, H, write_h)
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
  const unsigned g = blocks_for((long long)R * H);
  if (y_dt == kF32)
    dyt_add_kernel<float><<<g, 256, 0, st>>>(h, (const float*)y, ldy, p, R, H);
  else if (y_dt == kBF16)
    dyt_add_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(h, (const __nv_bfloat16*)y, ldy, p, R, H);
  else
    return kBadDType;
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
  const unsigned g = blocks_for((long long)T * H);
  if (out_dt == kF32)
    shift_rows_kernel<float><<<g, 256, 0, st>>>(h, p, shift, state, (size_t)state_stride, tok_seq,
                                                seq_slot, cu_seqlens, (float*)out, T, H);
  else if (out_dt == kBF16)
    shift_rows_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(h, p, shift, state, (size_t)state_stride,
                                                        tok_seq, seq_slot, cu_seqlens,
                                                        (__nv_bfloat16*)out, T, H);
  else
    return kBadDType;
  return launch_status();
}
