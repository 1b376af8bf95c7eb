// Whole-sequence LSTM / GRU forward for small hidden sizes (H <= 128), inference only.
//
// The step-by-step path launches a GEMM and several pointwise kernels per time step; for the small
// recurrent models of the reference (its examples use H = 128) a step is microseconds of math and
// the sequence is bound by launches.  Here one CTA owns one batch row for the whole sequence:
// thread g holds row g of W_hh (bf16 pairs) in registers, the hidden state lives in shared memory,
// the input projections x_t W_ih^T + b_ih for all steps come from one GEMM beforehand, and the
// value of the next step is prefetched while the current one is computed.
//
// Gate order and formulas follow crates/axonml-nn/src/layers/rnn.rs:292-416 (LSTM i,f,g,o) and
// :617-700 (GRU r,z,n with n = tanh(x_n + r * (W_hn h + b_hn))).
#include "common.cuh"

namespace {
using namespace ax;

template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

// G = 4: LSTM, G = 3: GRU.  HP = H rounded up to 32/64/128 (rows are zero-padded in registers).
template <int G, int HP, typename TO>
__global__ void __launch_bounds__(G * HP)
rnn_seq_kernel(const float* __restrict__ xproj, const __nv_bfloat16* __restrict__ w_hh, const float* __restrict__ b_hh,
               const float* __restrict__ h0, const float* __restrict__ c0, TO* __restrict__ out, float* __restrict__ h_last,
               float* __restrict__ c_last, int T, int H) {
  __shared__ float h_s[HP];
  __shared__ float gate_s[G * HP];
  const int b = blockIdx.x;
  const int g = threadIdx.x;                 // gate row gi*H + j for g < G*H
  const int GH = G * H;
  const bool active = g < GH;
  float2 w[HP / 2];
#pragma unroll
  for (int k = 0; k < HP / 2; ++k) {
    float lo = 0.f, hi = 0.f;
    if (active) {
      if (2 * k < H) lo = __bfloat162float(w_hh[(long)g * H + 2 * k]);
      if (2 * k + 1 < H) hi = __bfloat162float(w_hh[(long)g * H + 2 * k + 1]);
    }
    w[k] = make_float2(lo, hi);
  }
  const float bias = (active && b_hh != nullptr) ? b_hh[g] : 0.f;
  if (g < HP) h_s[g] = (g < H && h0 != nullptr) ? h0[(long)b * H + g] : 0.f;
  float c = (G == 4 && g < H && c0 != nullptr) ? c0[(long)b * H + g] : 0.f;
  const float* xp = xproj + (long)b * T * GH;
  float x_next = (active && T > 0) ? xp[g] : 0.f;
  float xr = 0.f, xz = 0.f, xn = 0.f;        // GRU: thread j < H also needs the three input projections of its unit
  __syncthreads();
  for (int t = 0; t < T; ++t) {
    const float x_cur = x_next;
    if (active && t + 1 < T) x_next = xp[(long)(t + 1) * GH + g];
    if (G == 3 && g < H) {
      xr = xp[(long)t * GH + g];
      xz = xp[(long)t * GH + H + g];
      xn = xp[(long)t * GH + 2 * H + g];
    }
    float acc = bias;
#pragma unroll
    for (int k = 0; k < HP / 2; ++k) acc = fmaf(w[k].x, h_s[2 * k], fmaf(w[k].y, h_s[2 * k + 1], acc));
    if (active) gate_s[g] = (G == 4) ? acc + x_cur : acc;      // GRU keeps the hidden part separate (n gate)
    __syncthreads();
    if (g < H) {
      float h_new;
      if (G == 4) {
        const float ig = sigmoidf_(gate_s[g]), fg = sigmoidf_(gate_s[H + g]);
        const float gg = tanhf(gate_s[2 * H + g]), og = sigmoidf_(gate_s[3 * H + g]);
        c = fg * c + ig * gg;
        h_new = og * tanhf(c);
      } else {
        const float r = sigmoidf_(xr + gate_s[g]);
        const float z = sigmoidf_(xz + gate_s[H + g]);
        const float n = tanhf(xn + r * gate_s[2 * H + g]);
        h_new = (1.f - z) * n + z * h_s[g];
      }
      store_out(out + ((long)b * T + t) * H + g, h_new);
      // every thread finished reading h_s for this step before the barrier above
      h_s[g] = h_new;
    }
    __syncthreads();
  }
  if (g < H) {
    if (h_last != nullptr) h_last[(long)b * H + g] = h_s[g];
    if (G == 4 && c_last != nullptr) c_last[(long)b * H + g] = c;
  }
}

template <int G, typename TO>
int launch_rnn(const float* xproj, const void* w_hh, const float* b_hh, const float* h0, const float* c0, void* out,
               float* h_last, float* c_last, int B, int T, int H, cudaStream_t stream) {
  const auto* w = (const __nv_bfloat16*)w_hh;
  if (H <= 32)
    rnn_seq_kernel<G, 32, TO><<<B, G * 32, 0, stream>>>(xproj, w, b_hh, h0, c0, (TO*)out, h_last, c_last, T, H);
  else if (H <= 64)
    rnn_seq_kernel<G, 64, TO><<<B, G * 64, 0, stream>>>(xproj, w, b_hh, h0, c0, (TO*)out, h_last, c_last, T, H);
  else
    rnn_seq_kernel<G, 128, TO><<<B, G * 128, 0, stream>>>(xproj, w, b_hh, h0, c0, (TO*)out, h_last, c_last, T, H);
  return (int)cudaGetLastError();
}

}  // namespace

// kind 4 = LSTM, 3 = GRU.  xproj: [B, T, kind*H] fp32 = x W_ih^T + b_ih; w_hh: [kind*H, H] bf16; b_hh: [kind*H] fp32 or
// null; h0 / c0: [B, H] fp32 or null (zeros); out: [B, T, H] (out_bf16 ? bf16 : fp32); h_last / c_last: [B, H] fp32 or null.
AX_API int ax_rnn_seq_fwd(int kind, const float* xproj, const void* w_hh, const float* b_hh, const float* h0,
                          const float* c0, void* out, int out_bf16, float* h_last, float* c_last, int B, int T, int H,
                          cudaStream_t stream) {
  if ((kind != 3 && kind != 4) || B <= 0 || T < 0 || H <= 0 || H > 128) return -1;
  if (T == 0) return 0;
  if (kind == 4)
    return out_bf16 ? launch_rnn<4, __nv_bfloat16>(xproj, w_hh, b_hh, h0, c0, out, h_last, c_last, B, T, H, stream)
                    : launch_rnn<4, float>(xproj, w_hh, b_hh, h0, c0, out, h_last, c_last, B, T, H, stream);
  return out_bf16 ? launch_rnn<3, __nv_bfloat16>(xproj, w_hh, b_hh, h0, c0, out, h_last, c_last, B, T, H, stream)
                  : launch_rnn<3, float>(xproj, w_hh, b_hh, h0, c0, out, h_last, c_last, B, T, H, stream);
}
