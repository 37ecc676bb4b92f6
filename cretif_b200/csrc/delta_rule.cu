// The gated delta rule: a matrix-valued recurrence per head, behind short causal convolutions.
//
// Per token and head, with state M [d, e] (32-bit, zero at a sequence's start):
//     M <- g M;   u = beta (v - M^T k);   M <- M + k u^T;   o = M^T q
// so the read-out sees the token's own write.  Three kernels serve any step shape (whole
// prompts, further chunks at a cached position, single tokens), all arithmetic in 32-bit:
//
// * delta_prepare (a CTA per token): the causal convolution over time of the projected q, k
//   and v channels (taps from this step's rows, or from the sequence's saved last inputs where
//   the window reaches back before the step), SiLU, unit length per q/k head (and the query's
//   d^-1/2), beta = sigmoid(.), g = exp(-exp(A_log) softplus(. + dt_bias)).
// * delta_recurrence (a CTA per (sequence, head)): the columns of M are independent, so a
//   group of P lanes owns one column, each lane a slice of its d rows in registers; a token
//   costs two P-lane shuffle reductions and no barrier.  Tokens go in chunks of 16 whose
//   operands are staged in shared memory; after a chunk the warps norm its outputs over e
//   (RMS, weight, times SiLU of the gate) and store them.  The state is read once and written
//   once per step.
// * delta_conv_state (a CTA per sequence): the last taps-1 inputs of every channel, for the
//   next step.
#include "api.h"
#include "common.cuh"

namespace cretif {

__device__ __forceinline__ float silu_f32(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f32(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// proj row: [q (G d) | k (G d) | v (H e) | gate (H e) | b (H) | a (H)]
// prep row: [q (G d) | k (G d) | v (H e) | beta (H) | g (H)]
__global__ void __launch_bounds__(256)
delta_prepare_kernel(const float* __restrict__ proj, int ldp, float* __restrict__ prep, int ldo,
                     const float* __restrict__ conv_w, int taps,
                     const float* __restrict__ conv_state, size_t state_stride,
                     const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                     const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                     const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int H,
                     int G, int d, int e, float unit_eps) {
  extern __shared__ float ch[];                  // the token's q, k, v channels after SiLU
  const int t = blockIdx.x;
  const int b = tok_seq[t];
  const int lt = tok_pos[t] - seq_start[b];      // tokens of this sequence before t in the step
  const int C = 2 * G * d + H * e;
  const float* st = conv_state + (size_t)seq_slot[b] * state_stride;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.f;
    for (int i = 0; i < taps; ++i) {             // i tokens back
      const float w = conv_w[(size_t)c * taps + (taps - 1 - i)];
      const float z = i <= lt ? proj[(size_t)(t - i) * ldp + c]
                              : st[(size_t)c * (taps - 1) + (taps - 1) - (i - lt)];
      acc = fmaf(w, z, acc);
    }
    ch[c] = silu_f32(acc);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  float* out = prep + (size_t)t * ldo;
  for (int head = warp; head < 2 * G; head += nwarps) {      // q heads, then k heads
    const float* x = ch + (size_t)head * d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) ss += x[i] * x[i];
    ss = warp_sum(ss);
    float f = 1.0f / sqrtf(ss + unit_eps);
    if (head < G) f *= 1.0f / sqrtf((float)d);
    for (int i = lane; i < d; i += 32) out[(size_t)head * d + i] = x[i] * f;
  }
  for (int i = threadIdx.x; i < H * e; i += blockDim.x) out[2 * G * d + i] = ch[2 * G * d + i];
  const float* row = proj + (size_t)t * ldp;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float bz = row[C + H * e + h], az = row[C + H * e + H + h];
    out[C + h] = 1.0f / (1.0f + expf(-bz));
    out[C + H + h] = expf(-expf(a_log[h]) * softplus_f32(az + dt_bias[h]));
  }
}

__global__ void delta_conv_state_kernel(const float* __restrict__ proj, int ldp,
                                        float* __restrict__ conv_state, size_t state_stride,
                                        int taps, int C, const int* __restrict__ cu_seqlens,
                                        const int* __restrict__ seq_slot) {
  const int b = blockIdx.x;
  const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
  float* st = conv_state + (size_t)seq_slot[b] * state_stride;
  const int keep = taps - 1;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float* s = st + (size_t)c * keep;
    for (int j = 0; j < keep; ++j) {             // ascending: reads run ahead of writes
      const int back = keep - j;                 // this entry is `back` tokens before the next
      s[j] = back <= n ? proj[(size_t)(t0 + n - back) * ldp + c] : s[j + n];
    }
  }
}

constexpr int kChunk = 16;

template <int DREG, typename TO>
__global__ void __launch_bounds__(1024)
delta_recurrence_kernel(const float* __restrict__ prep, int ldp, const float* __restrict__ gate,
                        int ldg, float* __restrict__ state, size_t state_stride,
                        const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                        int H, int G, int d, int e, int P, const float* __restrict__ norm_w,
                        float eps, TO* __restrict__ out, int ldo, int write_state) {
  extern __shared__ float sm[];
  const int b = blockIdx.x, h = blockIdx.y, grp = h / (H / G);
  const int dpad = P * DREG;
  float* qs = sm;                                // [kChunk][dpad]
  float* ks = qs + kChunk * dpad;                // [kChunk][dpad]
  float* vs = ks + kChunk * dpad;                // [kChunk][e]
  float* os = vs + kChunk * e;                   // [kChunk][e]
  float* bs = os + kChunk * e;                   // [kChunk] beta
  float* gs = bs + kChunk;                       // [kChunk] decay
  const int tid = threadIdx.x, part = tid % P, j = tid / P;
  const bool active = j < e;
  float* M = state + (size_t)seq_slot[b] * state_stride + (size_t)h * d * e;
  float S[DREG];
#pragma unroll
  for (int r = 0; r < DREG; ++r) {
    const int i = part + P * r;
    S[r] = (active && i < d) ? M[(size_t)i * e + j] : 0.f;
  }
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  const int C = 2 * G * d + H * e;
  const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
  for (int c0 = t0; c0 < t1; c0 += kChunk) {
    const int n = min(kChunk, t1 - c0);
    for (int idx = tid; idx < n * dpad; idx += blockDim.x) {
      const int tt = idx / dpad, i = idx - tt * dpad;
      const float* row = prep + (size_t)(c0 + tt) * ldp;
      qs[idx] = i < d ? row[(size_t)grp * d + i] : 0.f;
      ks[idx] = i < d ? row[(size_t)(G + grp) * d + i] : 0.f;
    }
    for (int idx = tid; idx < n * e; idx += blockDim.x) {
      const int tt = idx / e, i = idx - tt * e;
      vs[idx] = prep[(size_t)(c0 + tt) * ldp + 2 * G * d + (size_t)h * e + i];
    }
    if (tid < n) {
      bs[tid] = prep[(size_t)(c0 + tid) * ldp + C + h];
      gs[tid] = prep[(size_t)(c0 + tid) * ldp + C + H + h];
    }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const float* kk = ks + tt * dpad + part;
      const float* qq = qs + tt * dpad + part;
      const float g = gs[tt];
      float r = 0.f;
#pragma unroll
      for (int x = 0; x < DREG; ++x) r = fmaf(S[x], kk[P * x], r);
      for (int o = P >> 1; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
      const float u = bs[tt] * ((active ? vs[tt * e + j] : 0.f) - g * r);
      float acc = 0.f;
#pragma unroll
      for (int x = 0; x < DREG; ++x) {
        S[x] = fmaf(kk[P * x], u, g * S[x]);
        acc = fmaf(S[x], qq[P * x], acc);
      }
      for (int o = P >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (active && part == 0) os[tt * e + j] = acc;
    }
    __syncthreads();
    for (int tt = warp; tt < n; tt += nwarps) {       // the chunk's outputs, a warp per token
      const float* o = os + tt * e;
      float ss = 0.f;
      for (int i = lane; i < e; i += 32) ss += o[i] * o[i];
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)e + eps);
      const float* grow = gate + (size_t)(c0 + tt) * ldg + (size_t)h * e;
      TO* orow = out + (size_t)(c0 + tt) * ldo + (size_t)h * e;
      for (int i = lane; i < e; i += 32)
        orow[i] = from_float<TO>(o[i] * inv * norm_w[i] * silu_f32(grow[i]));
    }
    __syncthreads();
  }
  if (write_state) {
#pragma unroll
    for (int r = 0; r < DREG; ++r) {
      const int i = part + P * r;
      if (active && i < d) M[(size_t)i * e + j] = S[r];
    }
  }
}

template <int DREG, typename TO>
static int launch_recurrence(const float* prep, int ldp, const float* gate, int ldg, float* state,
                             size_t state_stride, const int* cu, const int* seq_slot, int B, int H,
                             int G, int d, int e, int P, const float* norm_w, float eps, void* out,
                             int ldo, int write_state, cudaStream_t st) {
  const int threads = ((e * P + 31) / 32) * 32;
  const size_t smem = sizeof(float) * ((size_t)kChunk * (2 * P * DREG + 2 * e) + 2 * kChunk);
  auto kern = delta_recurrence_kernel<DREG, TO>;
  if (smem > 48 * 1024) {
    if (smem > 200 * 1024) return kBadArgument;
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  kern<<<dim3(B, H), threads, smem, st>>>(prep, ldp, gate, ldg, state, state_stride, cu, seq_slot,
                                          H, G, d, e, P, norm_w, eps, (TO*)out, ldo, write_state);
  return launch_status();
}

}  // namespace cretif

using namespace cretif;

extern "C" int cretif_delta_prepare(const float* proj, int ldp, float* prep, int ldo,
                                    const float* conv_w, int taps, const float* conv_state,
                                    long long state_stride, const float* a_log,
                                    const float* dt_bias, const int* tok_pos, const int* tok_seq,
                                    const int* seq_slot, const int* seq_start, int H, int G, int d,
                                    int e, float unit_eps, int T, void* stream) {
  if (T <= 0) return kOk;
  if (H <= 0 || G <= 0 || H % G || d <= 0 || e <= 0 || taps < 1) return kBadArgument;
  const int C = 2 * G * d + H * e;
  if (ldp < C + H * e + 2 * H || ldo < C + 2 * H) return kBadArgument;
  const size_t smem = sizeof(float) * (size_t)C;
  if (smem > 200 * 1024) return kBadArgument;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(delta_prepare_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  delta_prepare_kernel<<<T, 256, smem, (cudaStream_t)stream>>>(
      proj, ldp, prep, ldo, conv_w, taps, conv_state, (size_t)state_stride, a_log, dt_bias,
      tok_pos, tok_seq, seq_slot, seq_start, H, G, d, e, unit_eps);
  return launch_status();
}

extern "C" int cretif_delta_conv_state(const float* proj, int ldp, float* conv_state,
                                       long long state_stride, int taps, int C,
                                       const int* cu_seqlens, const int* seq_slot, int B,
                                       void* stream) {
  if (B <= 0 || taps <= 1) return kOk;
  if (C <= 0 || ldp < C) return kBadArgument;
  delta_conv_state_kernel<<<B, 256, 0, (cudaStream_t)stream>>>(
      proj, ldp, conv_state, (size_t)state_stride, taps, C, cu_seqlens, seq_slot);
  return launch_status();
}

extern "C" int cretif_delta_recurrence(const float* prep, int ldp, const float* gate, int ldg,
                                       float* state, long long state_stride,
                                       const int* cu_seqlens, const int* seq_slot, int B, int H,
                                       int G, int d, int e, const float* norm_w, float eps,
                                       void* out, int out_dt, int ldo, int write_state,
                                       void* stream) {
  if (B <= 0) return kOk;
  if (H <= 0 || G <= 0 || H % G || d <= 0 || e <= 0 || e > 1024) return kBadArgument;
  // P lanes share a column: enough that a lane holds at most 32 rows, as long as the CTA
  // stays within 1024 threads; a lane then holds up to 128
  int P = 1;
  while (P < 32 && (d + P - 1) / P > 32 && ((e * 2 * P + 31) / 32) * 32 <= 1024) P *= 2;
  const int rows = (d + P - 1) / P;
  if (rows > 128) return kBadArgument;
  cudaStream_t st = (cudaStream_t)stream;
#define CRETIF_DELTA(DREG)                                                                        \
  (out_dt == kF32                                                                                 \
       ? launch_recurrence<DREG, float>(prep, ldp, gate, ldg, state, (size_t)state_stride,       \
                                        cu_seqlens, seq_slot, B, H, G, d, e, P, norm_w, eps, out, \
                                        ldo, write_state, st)                                     \
       : launch_recurrence<DREG, __nv_bfloat16>(prep, ldp, gate, ldg, state,                     \
                                                (size_t)state_stride, cu_seqlens, seq_slot, B, H, \
                                                G, d, e, P, norm_w, eps, out, ldo, write_state,   \
                                                st))
  if (out_dt != kF32 && out_dt != kBF16) return kBadDType;
  if (rows <= 8) return CRETIF_DELTA(8);
  if (rows <= 16) return CRETIF_DELTA(16);
  if (rows <= 32) return CRETIF_DELTA(32);
  if (rows <= 64) return CRETIF_DELTA(64);
  return CRETIF_DELTA(128);
#undef CRETIF_DELTA
}
