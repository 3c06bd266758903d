// Retention: linear attention with a fixed decay per head, no softmax and no denominator, over
// packed rows of several sequences, with the state carried per sequence.
//
//   q_t, k_t rotated by position on their first `rot` dimensions (pairs (i, i + rot/2)), k_t scaled;
//   S_t = decay_h * S_{t-1} + k_t v_t^T        (S: [dim][vdim] per head, float, zero at the start)
//   o_t = S_t^T q_t;   o_t / sqrt(mean(o_t^2) + eps) per head;   times silu(g_t)
//
// q, k, v, g are column ranges of one projection (row stride ld); everything after the projection
// is float: angles, sine and cosine, the rotated and scaled q and k, the state, the products with
// it, the per-head norm and the gate.  The result is stored in the activation type.
//
// This file holds the recurrent form: a block owns one (sequence, head) and walks the sequence's
// rows of the step in order, the state in registers (thread (s, c) holds rows s*RPT .. s*RPT+RPT-1
// of column c).  It serves decode steps, and prompts wherever the chunked form does not run; both
// do the same sums in a different order.
#include "common.cuh"

template <typename T, int RPT>
__global__ void __launch_bounds__(RPT >= 64 ? 1024 : 512) retention_recurrent_kernel(
    T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
    const T* __restrict__ g, int ld, float* __restrict__ state, const float* __restrict__ decay,
    const float* __restrict__ inv_freq, int rot, float k_scale, float eps,
    const int* __restrict__ seq_slot, const int* __restrict__ seq_pos0, const int* __restrict__ seq_qstart,
    const int* __restrict__ seq_qlen, int H, int d, int e) {
  extern __shared__ float sm[];
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.y, h = blockIdx.x;
  const int slot = seq_slot[b];
  const int n = seq_qlen ? seq_qlen[b] : 1;
  const int q0 = seq_qstart[b], pos0 = seq_pos0[b];
  const int DS = (d + RPT - 1) / RPT;
  const int tid = threadIdx.x;
  const int c = tid % e, s = tid / e;          // blockDim.x >= e * DS; threads with s >= DS hold no state
  const int r0 = s * RPT;
  float* qs = sm;                 // [d]
  float* ks = qs + d;             // [d]
  float* vs = ks + d;             // [e]
  float* part = vs + e;           // [DS][e]
  float* red = part + DS * e;     // [33]
  const float dec = decay[h];
  const int half = rot / 2;

  float S[RPT];
  float* sp = slot >= 0 ? state + (((size_t)slot * H + h) * d) * e : nullptr;
#pragma unroll
  for (int r = 0; r < RPT; r++) S[r] = (sp && r0 + r < d) ? sp[(size_t)(r0 + r) * e + c] : 0.f;

  for (int i = 0; i < n; i++) {
    const size_t m = (size_t)q0 + i;
    const float pos = (float)(pos0 + i);
    const T* qr = q + m * ld + (size_t)h * d;
    const T* kr = k + m * ld + (size_t)h * d;
    // rotated q and k of this row, and its v
    for (int j = tid; j < d; j += blockDim.x) {
      float qa = to_f32(qr[j]), ka = to_f32(kr[j]);
      if (j < rot) {
        const int p = j < half ? j : j - half;
        const float th = pos * inv_freq[p];
        const float cs = cosf(th), sn = sinf(th);
        const int jo = j < half ? j + half : j - half;
        const float qb = to_f32(qr[jo]), kb = to_f32(kr[jo]);
        if (j < half) { qa = qa * cs - qb * sn; ka = ka * cs - kb * sn; }
        else { qa = qa * cs + qb * sn; ka = ka * cs + kb * sn; }
      }
      qs[j] = qa;
      ks[j] = ka * k_scale;
    }
    for (int j = tid; j < e; j += blockDim.x) vs[j] = to_f32(v[m * ld + (size_t)h * e + j]);
    __syncthreads();
    const float vc = vs[c];
    float acc = 0.f;
#pragma unroll
    for (int r = 0; r < RPT; r++) {
      if (r0 + r < d) {
        S[r] = dec * S[r] + ks[r0 + r] * vc;
        acc += S[r] * qs[r0 + r];
      }
    }
    if (s < DS) part[s * e + c] = acc;
    __syncthreads();
    float o = 0.f;
    if (tid < e) {
      for (int ss = 0; ss < DS; ss++) o += part[ss * e + tid];
    }
    const float tot = block_sum(tid < e ? o * o : 0.f, red);    // syncs inside: qs, ks, vs and part are free again after it
    if (tid < e) {
      const float r = 1.0f / sqrtf(tot / (float)e + eps);
      const float gz = to_f32(g[m * ld + (size_t)h * e + tid]);
      out[m * (size_t)(H * e) + (size_t)h * e + tid] = from_f32<T>(o * r * (gz / (1.0f + expf(-gz))));
    }
  }
  if (sp) {
#pragma unroll
    for (int r = 0; r < RPT; r++)
      if (r0 + r < d) sp[(size_t)(r0 + r) * e + c] = S[r];
  }
}

template <typename T, int RPT>
static int launch_recurrent(void* out, const void* q, const void* k, const void* v, const void* g, int ld,
                            float* state, const float* decay, const float* inv_freq, int rot, float k_scale,
                            float eps, const int* seq_slot, const int* seq_pos0, const int* seq_qstart,
                            const int* seq_qlen, int B, int H, int d, int e, cudaStream_t st) {
  const int DS = ceil_div(d, RPT);
  const int threads = (e * DS + 31) / 32 * 32;      // whole warps; the spare threads only take part in the sums
  const size_t smem = (size_t)(2 * d + e + DS * e + 33) * sizeof(float);
  auto kern = retention_recurrent_kernel<T, RPT>;
  if (smem > 48 * 1024) {
    cudaError_t er = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (er != cudaSuccess) return leb_fail("leb_retention: shared memory %zu: %s", smem, cudaGetErrorString(er));
  }
  leb_launch(kern, dim3(H, B), dim3(threads), smem, st, (T*)out, (const T*)q, (const T*)k, (const T*)v,
             (const T*)g, ld, state, decay, inv_freq, rot, k_scale, eps, seq_slot, seq_pos0, seq_qstart, seq_qlen,
             H, d, e);
  LEB_CHECK_LAUNCH("leb_retention");
  return 0;
}

// out [M, H*e]; q, k [M, H*d], v, g [M, H*e] with row stride ld; state [slot][H][d][e] float;
// seq_qlen may be null for one row per sequence.
LEB_API int leb_retention(void* out, const void* q, const void* k, const void* v, const void* g, int ld, int dtype,
                          float* state, const float* decay, const float* inv_freq, int rot, float k_scale, float eps,
                          const int* seq_slot, const int* seq_pos0, const int* seq_qstart, const int* seq_qlen,
                          int M, int B, int H, int d, int e, cudaStream_t st) {
  if (M <= 0 || B <= 0) return 0;
  LEB_REQUIRE(dtype == LEB_F32 || dtype == LEB_BF16, "leb_retention: unknown dtype %d", dtype);
  LEB_REQUIRE(d >= 1 && e >= 1 && e <= 1024 && d <= 1024, "leb_retention: head sizes %d x %d outside 1..1024", d, e);
  LEB_REQUIRE(rot >= 0 && rot <= d && rot % 2 == 0, "leb_retention: %d rotated dimensions do not fit %d", rot, d);
  LEB_REQUIRE(B <= 65535, "leb_retention: %d sequences in one launch", B);
  // rows of the state per thread: the fewest that keep the block within 512 threads (1024 at most)
  int rpt = 4;
  while (rpt < 64 && e * ceil_div(d, rpt) > 512) rpt *= 2;
  LEB_REQUIRE(e * ceil_div(d, rpt) <= 1024, "leb_retention: a head of %d x %d is more than a block holds", d, e);
#define LEB_RET(T, R) launch_recurrent<T, R>(out, q, k, v, g, ld, state, decay, inv_freq, rot, k_scale, eps, seq_slot, \
                                             seq_pos0, seq_qstart, seq_qlen, B, H, d, e, st)
#define LEB_RET_T(T) (rpt == 4 ? LEB_RET(T, 4) : rpt == 8 ? LEB_RET(T, 8) : rpt == 16 ? LEB_RET(T, 16) \
                      : rpt == 32 ? LEB_RET(T, 32) : LEB_RET(T, 64))
  return dtype == LEB_F32 ? LEB_RET_T(float) : LEB_RET_T(bf16);
#undef LEB_RET_T
#undef LEB_RET
}
