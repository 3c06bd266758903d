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

// The same for 16 bytes of channels per thread (8 bfloat16 or 4 float) and CC_RT rows in a row: the
// taps and the last TAPS-1 rows stay in registers, every row is read once.  Sums in the scalar kernel's order.
constexpr int CC_RT = 8;
template <int VEC> __device__ __forceinline__ void load_vec(float* o, const float* p) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
template <int VEC> __device__ __forceinline__ void load_vec(float* o, const bf16* p) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const uint32_t r[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r[i]));
    o[2 * i] = f.x;
    o[2 * i + 1] = f.y;
  }
}
template <int VEC> __device__ __forceinline__ void store_vec(float* p, const float* a) {
  *reinterpret_cast<float4*>(p) = make_float4(a[0], a[1], a[2], a[3]);
}
template <int VEC> __device__ __forceinline__ void store_vec(bf16* p, const float* a) {
  uint32_t r[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
    r[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(r[0], r[1], r[2], r[3]);
}

template <typename T, int VEC, int TAPS>
__global__ void __launch_bounds__(128) causal_conv_rows_kernel(
    T* __restrict__ y, int ldy, const T* __restrict__ u, int ldu, const float* __restrict__ w,
    const float* __restrict__ state, const int* __restrict__ row_seq, const int* __restrict__ seq_slot,
    const int* __restrict__ seq_qstart, int M, int C) {
  pdl_trigger();
  pdl_wait();
  const int m0 = blockIdx.x * CC_RT;
  const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  if (c0 >= C) return;
  float wv[VEC][TAPS], win[TAPS - 1][VEC];
#pragma unroll
  for (int e = 0; e < VEC; e++)
#pragma unroll
    for (int j = 0; j < TAPS; j++) wv[e][j] = w[(size_t)(c0 + e) * TAPS + j];
#pragma unroll
  for (int r = 0; r < CC_RT; r++) {
    const int m = m0 + r;
    if (m >= M) break;
    const int b = row_seq[m];
    const int i = m - seq_qstart[b];
    if (r == 0 || i == 0) {      // the rows before this one: of this step, or the sequence's state
      const int slot = seq_slot[b];
#pragma unroll
      for (int j = 0; j < TAPS - 1; j++) {
        const int li = i - (TAPS - 1) + j;
        if (li >= 0) {
          load_vec<VEC>(win[j], u + (size_t)(m - i + li) * ldu + c0);
        } else {
#pragma unroll
          for (int e = 0; e < VEC; e++)
            win[j][e] = slot >= 0 ? state[((size_t)slot * C + c0 + e) * (TAPS - 1) + (TAPS - 1) + li] : 0.f;
        }
      }
    }
    float cur[VEC], acc[VEC];
    load_vec<VEC>(cur, u + (size_t)m * ldu + c0);
#pragma unroll
    for (int e = 0; e < VEC; e++) {
      float a = 0.f;
#pragma unroll
      for (int j = 0; j < TAPS - 1; j++) a += wv[e][j] * win[j][e];
      acc[e] = a + wv[e][TAPS - 1] * cur[e];
    }
    store_vec<VEC>(y + (size_t)m * ldy + c0, acc);
#pragma unroll
    for (int j = 0; j + 1 < TAPS - 1; j++)
#pragma unroll
      for (int e = 0; e < VEC; e++) win[j][e] = win[j + 1][e];
#pragma unroll
    for (int e = 0; e < VEC; e++) win[TAPS - 2][e] = cur[e];
  }
}

template <typename T, int VEC>
static bool launch_conv_rows(void* y, int ldy, const void* u, int ldu, const float* w, const float* state,
                             const int* row_seq, const int* seq_slot, const int* seq_qstart, int M, int C, int taps,
                             cudaStream_t st) {
  if (taps < 2 || taps > 5 || C % VEC != 0 || ((uintptr_t)y % 16) != 0 || ((uintptr_t)u % 16) != 0 ||
      ((size_t)ldy * sizeof(T)) % 16 != 0 || ((size_t)ldu * sizeof(T)) % 16 != 0)
    return false;
  const dim3 grid(ceil_div(M, CC_RT), ceil_div(C / VEC, 128)), block(128);
#define LEB_CCR(TAPS_) leb_launch(causal_conv_rows_kernel<T, VEC, TAPS_>, grid, block, 0, st, (T*)y, ldy, (const T*)u, ldu, w, \
                                  state, row_seq, seq_slot, seq_qstart, M, C)
  if (taps == 2) LEB_CCR(2);
  else if (taps == 3) LEB_CCR(3);
  else if (taps == 4) LEB_CCR(4);
  else LEB_CCR(5);
#undef LEB_CCR
  return true;
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
  float acc = 0.f;
  for (int s = 0; s < taps - 1; s++) {
    old[s] = sp ? sp[s] : 0.f;
    acc += w[(size_t)c * taps + s] * old[s];
  }
  acc += w[(size_t)c * taps + taps - 1] * un;      // oldest tap first, as the other forms sum
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
  const bool rows = dtype == LEB_F32
      ? launch_conv_rows<float, 4>(y, ldy, u, ldu, w, state, row_seq, seq_slot, seq_qstart, M, C, taps, st)
      : launch_conv_rows<bf16, 8>(y, ldy, u, ldu, w, state, row_seq, seq_slot, seq_qstart, M, C, taps, st);
  if (rows) {
    // 16 bytes of channels and several rows per thread
  } else if (dtype == LEB_F32)
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
