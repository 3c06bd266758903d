// A short causal depthwise convolution over time on the columns of a projection, for packed rows
// of several sequences, with the last taps-1 projected values of every sequence kept as state.
//
//   y[t, c] = sum_{j < taps} w[c, j] * u[t - (taps-1) + j, c],   u = 0 before the sequence's start
//
// No gate, no bias, no activation (the gated form of the convolution mixer is shortconv.cu).
// state [slot][C][taps-1] (float) holds u at the positions len-(taps-1) .. len-1 of the sequence in
// the slot, zero where the sequence has not got that far.  Products and sums are float.
//
// A step of several rows per sequence runs two kernels: the convolution (a thread per row and
// channel; rows before the step come from the state) and then the state's update (a thread per
// sequence and channel); a step of one row per sequence does both in one.
#include "common.cuh"

constexpr int CC_MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(128) causal_conv_kernel(
    T* __restrict__ y, int ldy, const T* __restrict__ u, int ldu, const float* __restrict__ w,
    const float* __restrict__ state, const int* __restrict__ row_seq, const int* __restrict__ seq_slot,
    const int* __restrict__ seq_qstart, int C, int taps) {
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = row_seq[m];
  const int slot = seq_slot[b];
  const int i = m - seq_qstart[b];          // the row's place among its sequence's rows of this step
  const float* sp = slot >= 0 ? state + ((size_t)slot * C + c) * (taps - 1) : nullptr;
  float acc = 0.f;
  for (int j = 0; j < taps; j++) {
    const int li = i - (taps - 1) + j;
    float v;
    if (li >= 0) v = to_f32(u[(size_t)(m - i + li) * ldu + c]);
    else v = sp ? sp[(taps - 1) + li] : 0.f;
    acc += w[(size_t)c * taps + j] * v;
  }
  y[(size_t)m * ldy + c] = from_f32<T>(acc);
}

// After the convolution: the state moves on by the sequence's rows of this step.
template <typename T>
__global__ void __launch_bounds__(128) causal_conv_state_kernel(
    const T* __restrict__ u, int ldu, float* __restrict__ state, const int* __restrict__ seq_slot,
    const int* __restrict__ seq_qstart, const int* __restrict__ seq_qlen, int C, int taps) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int slot = seq_slot[b];
  if (slot < 0) return;
  const int n = seq_qlen[b], q0 = seq_qstart[b];
  float* sp = state + ((size_t)slot * C + c) * (taps - 1);
  for (int s = 0; s < taps - 1; s++) {       // ascending: an old value is read before its place is written
    const int li = n - (taps - 1) + s;
    sp[s] = li >= 0 ? to_f32(u[(size_t)(q0 + li) * ldu + c]) : sp[s + n];
  }
}

// One row per sequence: convolution and update by the same thread.
template <typename T>
__global__ void __launch_bounds__(128) causal_conv_single_kernel(
    T* __restrict__ y, int ldy, const T* __restrict__ u, int ldu, const float* __restrict__ w,
    float* __restrict__ state, const int* __restrict__ seq_slot, const int* __restrict__ seq_qstart, int C, int taps) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int slot = seq_slot[b];
  const int m = seq_qstart[b];
  const float un = to_f32(u[(size_t)m * ldu + c]);
  float* sp = slot >= 0 ? state + ((size_t)slot * C + c) * (taps - 1) : nullptr;
  float old[CC_MAX_TAPS];
  float acc = w[(size_t)c * taps + taps - 1] * un;
  for (int s = 0; s < taps - 1; s++) {
    old[s] = sp ? sp[s] : 0.f;
    acc += w[(size_t)c * taps + s] * old[s];
  }
  y[(size_t)m * ldy + c] = from_f32<T>(acc);
  if (sp) {
    for (int s = 0; s + 1 < taps - 1; s++) sp[s] = old[s + 1];
    if (taps > 1) sp[taps - 2] = un;
  }
}

LEB_API int leb_causal_conv(void* y, int ldy, const void* u, int ldu, int dtype, const float* w, float* state,
                            const int* row_seq, const int* seq_slot, const int* seq_qstart, const int* seq_qlen,
                            int M, int B, int C, int taps, int single, cudaStream_t st) {
  if (M <= 0 || C <= 0) return 0;
  LEB_REQUIRE(taps >= 1 && taps <= CC_MAX_TAPS, "leb_causal_conv: %d taps outside 1..%d", taps, CC_MAX_TAPS);
  LEB_REQUIRE(dtype == LEB_F32 || dtype == LEB_BF16, "leb_causal_conv: unknown dtype %d", dtype);
  LEB_REQUIRE(B <= 65535 && C <= 65535 * 128, "leb_causal_conv: step too large");
  dim3 block(128);
  const unsigned gx = (unsigned)ceil_div(C, 128);
  if (single) {
    LEB_REQUIRE(M == B, "leb_causal_conv: the single-row form needs one row per sequence");
    if (dtype == LEB_F32)
      leb_launch(causal_conv_single_kernel<float>, dim3(gx, B), block, 0, st, (float*)y, ldy, (const float*)u, ldu, w,
                 state, seq_slot, seq_qstart, C, taps);
    else
      leb_launch(causal_conv_single_kernel<bf16>, dim3(gx, B), block, 0, st, (bf16*)y, ldy, (const bf16*)u, ldu, w,
                 state, seq_slot, seq_qstart, C, taps);
    LEB_CHECK_LAUNCH("leb_causal_conv");
    return 0;
  }
  if (dtype == LEB_F32)
    leb_launch(causal_conv_kernel<float>, dim3(M, gx), block, 0, st, (float*)y, ldy, (const float*)u, ldu, w,
               (const float*)state, row_seq, seq_slot, seq_qstart, C, taps);
  else
    leb_launch(causal_conv_kernel<bf16>, dim3(M, gx), block, 0, st, (bf16*)y, ldy, (const bf16*)u, ldu, w,
               (const float*)state, row_seq, seq_slot, seq_qstart, C, taps);
  LEB_CHECK_LAUNCH("leb_causal_conv");
  if (taps > 1) {
    if (dtype == LEB_F32)
      leb_launch(causal_conv_state_kernel<float>, dim3(gx, B), block, 0, st, (const float*)u, ldu, state, seq_slot,
                 seq_qstart, seq_qlen, C, taps);
    else
      leb_launch(causal_conv_state_kernel<bf16>, dim3(gx, B), block, 0, st, (const bf16*)u, ldu, state, seq_slot,
                 seq_qstart, seq_qlen, C, taps);
    LEB_CHECK_LAUNCH("leb_causal_conv state");
  }
  return 0;
}
