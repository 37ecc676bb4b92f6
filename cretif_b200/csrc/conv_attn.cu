// What stands between an attention's projections and its scores when the projections pass a
// short causal convolution over time: convolution, unit length per head, a gain on the query
// that grows with the position, and the write into the block cache -- one kernel, 32-bit.
//
// proj rows (float32): [q (nh hd) | k (nkv hd) | v (nkv vd)]; a layer that reads another layer's
// keys and values has only the q columns (nkv = 0 here).  Channel c of a row is convolved with
// taps weights conv_w[c, :] (the last one for the present token) over this step's earlier rows of
// the same sequence and, where the window reaches back before the step, over the sequence's saved
// last taps-1 inputs (conv_state, [C, taps-1] per slot, zeros at a sequence's start).  Then
//   q head:  x / sqrt(mean(x^2) + eps) * (1 + coef * ln(floor((pos + 1) / every) + 1))  -> q_out
//   k head:  x / sqrt(mean(x^2) + eps)                                                  -> key cache
//   v head:  x                                                                          -> value cache
// A warp per head of a token (with many tokens, eight warps per token that take its heads in
// turn); a head's channels stay in the lanes' registers between the convolution and the scaling
// (head sizes up to 512).  The saved inputs are brought up to date
// afterwards by delta_conv_state (delta_rule.cu), which is the same for every convolved mixer.
#include "api.h"
#include "common.cuh"

namespace cretif {

namespace {
constexpr int kCvWarps = 8;
constexpr int kCvMaxD = 512;

// NCH: channels a lane keeps (head sizes up to 32 NCH).  TAPS: the number of taps when it is 2,
// 3 or 4 (the loops over them are then unrolled exactly), 0 for any number.
template <typename T, int NCH, int TAPS>
__global__ void __launch_bounds__(kCvWarps * 32)
conv_headnorm_kv_append_kernel(const float* __restrict__ proj, int ldp,
                               const float* __restrict__ conv_w, int taps,
                               const float* __restrict__ conv_state, size_t state_stride,
                               const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                               const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                               int nh, int nkv, int hd, int vd, float eps, float gain_coef,
                               int gain_every, T* __restrict__ q_out, int ldq,
                               const int* __restrict__ table, int table_stride,
                               T* __restrict__ kc, T* __restrict__ vc, int bt, int write_cache,
                               unsigned int* __restrict__ fault) {
  if (TAPS > 0) taps = TAPS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int units = nh + 2 * nkv;
  // what the token's heads share is read once; a warp then takes heads in turn (with many
  // tokens a CTA's eight warps take all of a token's heads: the chain of index loads is paid
  // once per warp and there are few enough warps to be resident together)
  const int b = tok_seq[t];
  const int pos = tok_pos[t];
  const int lt = pos - seq_start[b];             // tokens of this sequence before t in the step
  const int slot = seq_slot[b];
  const float* st = conv_state + (size_t)slot * state_stride;
  const float* row = proj + (size_t)t * ldp;
  int blk = 0;
  if (nkv > 0 && write_cache) {
    blk = table[(size_t)slot * table_stride + pos / bt];
    if (blk < 0) {
      if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(fault, kFaultBlockTable);
    }
  }
  const float gain =
      gain_every > 0 ? 1.0f + gain_coef * logf((float)((pos + 1) / gain_every + 1)) : 1.0f;
  // Where tap j (0 = the oldest) of channel c comes from is the same for every channel: this
  // step's row `back` tokens up, or the sequence's saved inputs; a base and a stride per tap.
  constexpr int kFastTaps = TAPS > 0 ? TAPS : 8;
  const float* tap_base[kFastTaps];
  int tap_stride[kFastTaps];
#pragma unroll
  for (int j = 0; j < kFastTaps; ++j) {
    const int back = taps - 1 - j;                // tokens back
    const bool here = back <= lt;
    tap_base[j] = here ? row - (ptrdiff_t)back * ldp : st + (taps - 1) - (back - lt);
    tap_stride[j] = here ? 1 : taps - 1;
  }
  auto conv = [&](int c) {
    float acc = 0.f;
    const float* w = conv_w + (size_t)c * taps;
    if (taps <= kFastTaps) {
#pragma unroll
      for (int j = 0; j < kFastTaps; ++j)
        if (j < taps) acc = fmaf(w[j], tap_base[j][(size_t)c * tap_stride[j]], acc);
      return acc;
    }
    for (int i = taps - 1; i >= 0; --i) {        // i tokens back, the oldest first
      const float z = i <= lt ? row[c - (ptrdiff_t)i * ldp]
                              : st[(size_t)c * (taps - 1) + (taps - 1) - (i - lt)];
      acc = fmaf(w[taps - 1 - i], z, acc);
    }
    return acc;
  };
  for (int unit = blockIdx.y * kCvWarps + warp; unit < units; unit += gridDim.y * kCvWarps) {
    const bool is_q = unit < nh, is_k = !is_q && unit < nh + nkv;
    const int n = (is_q || is_k) ? hd : vd;
    const int c0 = is_q ? unit * hd : is_k ? nh * hd + (unit - nh) * hd
                                           : (nh + nkv) * hd + (unit - nh - nkv) * vd;
    float val[NCH];
    float ss = 0.f;
#pragma unroll
    for (int m = 0; m < NCH; ++m) {
      const int i = lane + 32 * m;
      val[m] = i < n ? conv(c0 + i) : 0.f;
      ss += val[m] * val[m];
    }
    float f = 1.f;
    if (is_q || is_k) {
      ss = warp_sum(ss);
      f = 1.0f / sqrtf(ss / (float)hd + eps);
    }
    T* dst;
    if (is_q) {
      f *= gain;
      dst = q_out + (size_t)t * ldq + (size_t)unit * hd;
    } else {
      if (!write_cache || blk < 0) continue;
      const int kvh = is_k ? unit - nh : unit - nh - nkv;
      dst = (is_k ? kc : vc) + (((size_t)blk * nkv + kvh) * bt + (pos % bt)) * n;
    }
#pragma unroll
    for (int m = 0; m < NCH; ++m) {
      const int i = lane + 32 * m;
      if (i < n) dst[i] = from_float<T>(val[m] * f);
    }
  }
}
}  // namespace
}  // namespace cretif

using namespace cretif;

extern "C" int cretif_conv_headnorm_kv_append(
    const float* proj, int ldp, const float* conv_w, int taps, const float* conv_state,
    long long state_stride, const int* tok_pos, const int* tok_seq, const int* seq_slot,
    const int* seq_start, int nh, int nkv, int hd, int vd, float eps, float gain_coef,
    int gain_every, void* q_out, int ldq, int dt, const int* table, int table_stride, void* kc,
    void* vc, int bt, int write_cache, int T, unsigned int* fault, void* stream) {
  if (T <= 0) return kOk;
  if (nh <= 0 || nkv < 0 || hd <= 0 || hd > kCvMaxD || taps < 1 || ldq < nh * hd)
    return kBadArgument;
  if (nkv > 0 && (vd <= 0 || vd > kCvMaxD || bt <= 0 || !kc || !vc || !table)) return kBadArgument;
  if (ldp < (nh + nkv) * hd + nkv * vd) return kBadArgument;
  if (taps > 1 && !conv_state) return kBadArgument;
  const int units = nh + 2 * nkv;
  // few tokens: a warp per head, spread over CTAs; many: a CTA per token walks its heads
  dim3 grid(T, T >= 256 ? 1 : (units + kCvWarps - 1) / kCvWarps);
  if (grid.y > 65535) return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
  const int widest = nkv > 0 && vd > hd ? vd : hd;
#define CRETIF_CONV_K(TT, NCH, TAPS)                                                            \
  conv_headnorm_kv_append_kernel<TT, NCH, TAPS><<<grid, kCvWarps * 32, 0, st>>>(                 \
      proj, ldp, conv_w, taps, conv_state, (size_t)state_stride, tok_pos, tok_seq, seq_slot,     \
      seq_start, nh, nkv, hd, vd, eps, gain_coef, gain_every, (TT*)q_out, ldq, table,            \
      table_stride, (TT*)kc, (TT*)vc, bt, write_cache, fault)
#define CRETIF_CONV(TT, NCH)                                                                    \
  do {                                                                                          \
    if (taps == 4) CRETIF_CONV_K(TT, NCH, 4);                                                    \
    else if (taps == 3) CRETIF_CONV_K(TT, NCH, 3);                                               \
    else if (taps == 2) CRETIF_CONV_K(TT, NCH, 2);                                               \
    else CRETIF_CONV_K(TT, NCH, 0);                                                              \
  } while (0)
#define CRETIF_CONV_T(TT)                                                                       \
  do {                                                                                          \
    if (widest <= 64) CRETIF_CONV(TT, 2);                                                        \
    else if (widest <= 128) CRETIF_CONV(TT, 4);                                                  \
    else if (widest <= 256) CRETIF_CONV(TT, 8);                                                  \
    else CRETIF_CONV(TT, 16);                                                                    \
  } while (0)
  if (dt == kF32)
    CRETIF_CONV_T(float);
  else if (dt == kBF16)
    CRETIF_CONV_T(__nv_bfloat16);
  else
    return kBadDType;
#undef CRETIF_CONV_T
#undef CRETIF_CONV
#undef CRETIF_CONV_K
  return launch_status();
}
