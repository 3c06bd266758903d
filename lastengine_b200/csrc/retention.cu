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

// ---------------------------------------------------------------------------------------------
// The chunked form, for steps with many rows per sequence.  A sequence's rows are cut into chunks
// of RC rows.  With g = decay, L the rows of chunk c and S_c the state before its first row:
//   U_c = sum_j g^(L-1-j) k_j v_j^T                                   (kernel 1, every chunk at once)
//   S_{c+1} = g^L S_c + U_c, S_0 = the sequence's state               (kernel 2, a thread per state element)
//   o_i = sum_{j<=i} g^(i-j) (q_i . k_j) v_j + g^(i+1) S_c^T q_i      (kernel 3, every chunk at once)
// followed by the per-head norm and the gate as in the recurrent form.  All of it is float on the
// CUDA cores: scores, decay powers (by repeated multiplication, as the recurrence forms them),
// state and sums; only the order of the sums differs from the recurrent form.
constexpr int RC = 64;            // rows of a chunk
constexpr int RCT = 256;          // threads of a chunk's block

// (sequence, chunk within it, first row, rows) of chunk number `gidx` of the step, or false past the last
__device__ __forceinline__ bool find_chunk(int gidx, const int* seq_qlen, int B, int& b, int& c, int& nrows, int& base) {
  int acc = 0;
  for (int s = 0; s < B; s++) {
    const int n = seq_qlen[s];
    const int nc = (n + RC - 1) / RC;
    if (gidx < acc + nc) {
      b = s;
      c = gidx - acc;
      nrows = min(RC, n - c * RC);
      base = acc;
      return true;
    }
    acc += nc;
  }
  return false;
}

// Rotated q and k (k scaled, and weighted by wk[j] if given) and v of a chunk into shared memory,
// rows past the chunk's end as zeros.  ldq/ldv: padded row lengths in shared memory.
template <typename T>
__device__ __forceinline__ void stage_chunk(float* qs, float* ks, float* vs, int ldq, int ldv, const T* q, const T* k,
                                            const T* v, int ld, size_t row0, int nrows, int pos0, int h, int d, int e,
                                            const float* inv_freq, int rot, float k_scale, const float* wk) {
  const int half = rot / 2;
  const int npair = half + (d - rot);       // rotated pairs, then the dimensions that pass unchanged
  for (int idx = threadIdx.x; idx < RC * npair; idx += blockDim.x) {
    const int i = idx / npair, p = idx - i * npair;
    const bool in = i < nrows;
    const T* qr = q + (row0 + i) * ld + (size_t)h * d;
    const T* kr = k + (row0 + i) * ld + (size_t)h * d;
    const float w = k_scale * (wk ? wk[i] : 1.f);
    if (p < half) {
      float qa = 0.f, qb = 0.f, ka = 0.f, kb = 0.f;
      if (in) {
        float sn, cs;
        sincosf((float)(pos0 + i) * inv_freq[p], &sn, &cs);
        const float a = to_f32(qr[p]), bb = to_f32(qr[p + half]), a2 = to_f32(kr[p]), b2 = to_f32(kr[p + half]);
        qa = a * cs - bb * sn;
        qb = bb * cs + a * sn;
        ka = (a2 * cs - b2 * sn) * w;
        kb = (b2 * cs + a2 * sn) * w;
      }
      if (qs) { qs[i * ldq + p] = qa; qs[i * ldq + p + half] = qb; }
      ks[i * ldq + p] = ka;
      ks[i * ldq + p + half] = kb;
    } else {
      const int j = rot + (p - half);
      if (qs) qs[i * ldq + j] = in ? to_f32(qr[j]) : 0.f;
      ks[i * ldq + j] = in ? to_f32(kr[j]) * w : 0.f;
    }
  }
  for (int idx = threadIdx.x; idx < RC * e; idx += blockDim.x) {
    const int i = idx / e, j = idx - i * e;
    vs[i * ldv + j] = i < nrows ? to_f32(v[(row0 + i) * ld + (size_t)h * e + j]) : 0.f;
  }
}

// Kernel 1: U_c [d][e] of every chunk.  scratch [chunk][H][d][e].
template <typename T>
__global__ void __launch_bounds__(RCT) retention_chunk_state_kernel(
    float* __restrict__ scratch, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int ld,
    const float* __restrict__ decay, const float* __restrict__ inv_freq, int rot, float k_scale,
    const int* __restrict__ seq_pos0, const int* __restrict__ seq_qstart, const int* __restrict__ seq_qlen,
    int B, int H, int d, int e) {
  extern __shared__ float sm[];
  pdl_trigger();
  pdl_wait();
  int b, c, nrows, base;
  if (!find_chunk(blockIdx.x, seq_qlen, B, b, c, nrows, base)) return;
  const int h = blockIdx.y;
  const int d8 = (d + 7) & ~7, e8 = (e + 7) & ~7;
  float* ks = sm;                    // [RC][d8]
  float* vs = ks + RC * d8;          // [RC][e8]
  float* wk = vs + RC * e8;          // [RC]  g^(L-1-j)
  const float g = decay[h];
  if (threadIdx.x == 0) {
    float p = 1.f;
    for (int j = nrows - 1; j >= 0; j--) { wk[j] = p; p *= g; }
    for (int j = nrows; j < RC; j++) wk[j] = 0.f;
  }
  for (int idx = threadIdx.x; idx < RC * (d8 - d); idx += blockDim.x) ks[(idx / (d8 - d)) * d8 + d + idx % (d8 - d)] = 0.f;
  for (int idx = threadIdx.x; idx < RC * (e8 - e); idx += blockDim.x) vs[(idx / (e8 - e)) * e8 + e + idx % (e8 - e)] = 0.f;
  __syncthreads();
  stage_chunk<T>(nullptr, ks, vs, d8, e8, q, k, v, ld, (size_t)seq_qstart[b] + (size_t)c * RC, nrows,
                 seq_pos0[b] + c * RC, h, d, e, inv_freq, rot, k_scale, wk);
  __syncthreads();
  float* out = scratch + ((size_t)(base + c) * H + h) * d * e;
  const int te = e8 / 8, tiles = (d8 / 8) * te;
  // a thread's eight columns are two groups of four, half a row apart: neighbouring threads then read
  // neighbouring 16 bytes of shared memory
  for (int t = threadIdx.x; t < tiles; t += blockDim.x) {
    const int r0 = (t / te) * 8, ca = (t % te) * 4, cb = e8 / 2 + ca;
    float acc[8][8];
#pragma unroll
    for (int a = 0; a < 8; a++)
#pragma unroll
      for (int bb = 0; bb < 8; bb++) acc[a][bb] = 0.f;
    for (int j = 0; j < nrows; j++) {
      const float4 k0 = *reinterpret_cast<const float4*>(ks + j * d8 + r0), k1 = *reinterpret_cast<const float4*>(ks + j * d8 + r0 + 4);
      const float4 v0 = *reinterpret_cast<const float4*>(vs + j * e8 + ca), v1 = *reinterpret_cast<const float4*>(vs + j * e8 + cb);
      const float kk[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
      const float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
      for (int a = 0; a < 8; a++)
#pragma unroll
        for (int bb = 0; bb < 8; bb++) acc[a][bb] += kk[a] * vv[bb];
    }
#pragma unroll
    for (int a = 0; a < 8; a++)
#pragma unroll
      for (int bb = 0; bb < 8; bb++) {
        const int cc = bb < 4 ? ca + bb : cb + bb - 4;
        if (r0 + a < d && cc < e) out[(size_t)(r0 + a) * e + cc] = acc[a][bb];
      }
  }
}

// Kernel 2: the states before every chunk, in place of the U_c, and the sequence's state after the step.
__global__ void __launch_bounds__(256) retention_chunk_scan_kernel(
    float* __restrict__ scratch, float* __restrict__ state, const float* __restrict__ decay,
    const int* __restrict__ seq_slot, const int* __restrict__ seq_qlen, int B, int H, int de) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.z, h = blockIdx.y;
  const int x = blockIdx.x * blockDim.x + threadIdx.x;
  if (x >= de) return;
  int base = 0;
  for (int s = 0; s < b; s++) base += (seq_qlen[s] + RC - 1) / RC;
  const int n = seq_qlen[b], nc = (n + RC - 1) / RC;
  const int slot = seq_slot[b];
  const float g = decay[h];
  float gl = 1.f;                                  // g^RC, by repeated multiplication
  for (int j = 0; j < RC; j++) gl *= g;
  float* sp = slot >= 0 ? state + ((size_t)slot * H + h) * de + x : nullptr;
  float S = sp ? *sp : 0.f;
  const size_t step = (size_t)H * de;                       // from one chunk's element to the next chunk's
  float* u0 = scratch + ((size_t)base * H + h) * de + x;
  const int last = n - (nc - 1) * RC;                       // rows of the last chunk
  float glast = 1.f;
  for (int j = 0; j < last; j++) glast *= g;
  // eight chunks' sums are asked for before any is used: the loads do not depend on the running state
  for (int c0 = 0; c0 < nc; c0 += 8) {
    float U[8];
#pragma unroll
    for (int j = 0; j < 8; j++) U[j] = c0 + j < nc ? u0[(size_t)(c0 + j) * step] : 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      if (c0 + j < nc) {
        u0[(size_t)(c0 + j) * step] = S;
        S = (c0 + j == nc - 1 ? glast : gl) * S + U[j];
      }
    }
  }
  if (sp) *sp = S;
}

// Kernel 3: the chunk's outputs.
template <typename T>
__global__ void __launch_bounds__(RCT) retention_chunk_out_kernel(
    T* __restrict__ out, const float* __restrict__ scratch, const T* __restrict__ q, const T* __restrict__ k,
    const T* __restrict__ v, const T* __restrict__ gt, int ld, const float* __restrict__ decay,
    const float* __restrict__ inv_freq, int rot, float k_scale, float eps, const int* __restrict__ seq_pos0,
    const int* __restrict__ seq_qstart, const int* __restrict__ seq_qlen, int B, int H, int d, int e) {
  extern __shared__ float sm[];
  pdl_trigger();
  pdl_wait();
  int b, c, nrows, base;
  if (!find_chunk(blockIdx.x, seq_qlen, B, b, c, nrows, base)) return;
  const int h = blockIdx.y;
  const int d8 = (d + 7) & ~7, e8 = (e + 7) & ~7;
  float* qs = sm;                    // [RC][d8]
  float* ks = qs + RC * d8;          // [RC][d8], later slabs of the state [rows][e8]
  float* vs = ks + RC * d8;          // [RC][e8]
  float* as = vs + RC * e8;          // [RC][RC + 1] decayed scores
  float* pw = as + RC * (RC + 1);    // [RC + 1] powers of the decay
  const float g = decay[h];
  if (threadIdx.x == 0) {
    float p = 1.f;
    for (int j = 0; j <= RC; j++) { pw[j] = p; p *= g; }
  }
  for (int idx = threadIdx.x; idx < RC * (d8 - d); idx += blockDim.x) {
    const int o = (idx / (d8 - d)) * d8 + d + idx % (d8 - d);
    qs[o] = 0.f;
    ks[o] = 0.f;
  }
  for (int idx = threadIdx.x; idx < RC * (e8 - e); idx += blockDim.x) vs[(idx / (e8 - e)) * e8 + e + idx % (e8 - e)] = 0.f;
  const size_t row0 = (size_t)seq_qstart[b] + (size_t)c * RC;
  stage_chunk<T>(qs, ks, vs, d8, e8, q, k, v, ld, row0, nrows, seq_pos0[b] + c * RC, h, d, e, inv_freq, rot, k_scale,
                 nullptr);
  __syncthreads();
  // decayed scores A[i][j] = (q_i . k_j) g^(i-j), j <= i: a thread takes 4 x 4 of them
  {
    const int i0 = (threadIdx.x / 16) * 4, j0 = (threadIdx.x % 16) * 4;
    float acc[4][4] = {};
    if (j0 <= i0 + 3) {
      for (int r = 0; r < d8; r += 4) {
        float4 qa[4], kb[4];
#pragma unroll
        for (int a = 0; a < 4; a++) {
          qa[a] = *reinterpret_cast<const float4*>(qs + (i0 + a) * d8 + r);
          kb[a] = *reinterpret_cast<const float4*>(ks + (j0 + a) * d8 + r);
        }
#pragma unroll
        for (int a = 0; a < 4; a++)
#pragma unroll
          for (int bb = 0; bb < 4; bb++)
            acc[a][bb] += qa[a].x * kb[bb].x + qa[a].y * kb[bb].y + qa[a].z * kb[bb].z + qa[a].w * kb[bb].w;
      }
    }
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
      for (int bb = 0; bb < 4; bb++) {
        const int i = i0 + a, j = j0 + bb;
        as[i * (RC + 1) + j] = j <= i ? acc[a][bb] * pw[i - j] : 0.f;
      }
  }
  __syncthreads();       // the scores are written, and nobody reads ks any more: it takes the state's slabs
  // o[i][c] for a thread's 4 rows x 8 columns per tile: the chunk's own keys, then the state before the chunk
  const int te = e8 / 8, tiles = (RC / 4) * te;
  const float* Sg = scratch + ((size_t)(base + c) * H + h) * d * e;
  const int slab = max(1, min(d, (RC * d8) / e8));          // rows of the state that fit where ks was
  float acc[2][4][8];                                        // up to two tiles per thread (e <= 256: tiles <= 512)
#pragma unroll
  for (int u = 0; u < 2; u++)
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
      for (int bb = 0; bb < 8; bb++) acc[u][a][bb] = 0.f;
#pragma unroll
  for (int u = 0; u < 2; u++) {
    const int t = threadIdx.x + u * RCT;
    if (t >= tiles) break;
    const int i0 = (t / te) * 4, ca = (t % te) * 4, cb = e8 / 2 + ca;      // columns as in the state kernel
    for (int j = 0; j < min(nrows, i0 + 4); j++) {
      const float4 v0 = *reinterpret_cast<const float4*>(vs + j * e8 + ca), v1 = *reinterpret_cast<const float4*>(vs + j * e8 + cb);
      const float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
      for (int a = 0; a < 4; a++) {
        const float s = as[(i0 + a) * (RC + 1) + j];
#pragma unroll
        for (int bb = 0; bb < 8; bb++) acc[u][a][bb] += s * vv[bb];
      }
    }
  }
  // the rows of q times their power of the decay, once, so that the state's part is a plain product
  for (int idx = threadIdx.x; idx < RC * d8; idx += blockDim.x) qs[idx] *= pw[idx / d8 + 1];
  for (int r0 = 0; r0 < d; r0 += slab) {
    const int nr = min(slab, d - r0);
    __syncthreads();
    if ((e & 3) == 0) {          // 16-byte pieces of the state's rows
      const int q4 = e8 / 4;
      for (int idx = threadIdx.x; idx < nr * q4; idx += blockDim.x) {
        const int r = idx / q4, c4 = idx - r * q4;
        reinterpret_cast<float4*>(ks)[idx] = 4 * c4 < e ? *reinterpret_cast<const float4*>(Sg + (size_t)(r0 + r) * e + 4 * c4)
                                                        : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    } else {
      for (int idx = threadIdx.x; idx < nr * e8; idx += blockDim.x) {
        const int r = idx / e8, cc = idx - r * e8;
        ks[idx] = cc < e ? Sg[(size_t)(r0 + r) * e + cc] : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < 2; u++) {
      const int t = threadIdx.x + u * RCT;
      if (t >= tiles) break;
      const int i0 = (t / te) * 4, ca = (t % te) * 4, cb = e8 / 2 + ca;
      for (int r = 0; r < nr; r++) {
        const float4 s0 = *reinterpret_cast<const float4*>(ks + r * e8 + ca), s1 = *reinterpret_cast<const float4*>(ks + r * e8 + cb);
        const float ss[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int a = 0; a < 4; a++) {
          const float qv = qs[(i0 + a) * d8 + r0 + r];
#pragma unroll
          for (int bb = 0; bb < 8; bb++) acc[u][a][bb] += qv * ss[bb];
        }
      }
    }
  }
  __syncthreads();       // everyone is done with vs: the outputs go there, [RC][e8]
#pragma unroll
  for (int u = 0; u < 2; u++) {
    const int t = threadIdx.x + u * RCT;
    if (t >= tiles) break;
    const int i0 = (t / te) * 4, ca = (t % te) * 4, cb = e8 / 2 + ca;
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
      for (int bb = 0; bb < 8; bb++) vs[(i0 + a) * e8 + (bb < 4 ? ca + bb : cb + bb - 4)] = acc[u][a][bb];
  }
  __syncthreads();
  // per row: the head's root mean square, the gate, the store
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = warp; i < nrows; i += RCT / 32) {
    float ssq = 0.f;
    for (int j = lane; j < e; j += 32) ssq += vs[i * e8 + j] * vs[i * e8 + j];
    ssq = warp_sum(ssq);
    const float r = 1.0f / sqrtf(ssq / (float)e + eps);
    const size_t m = row0 + i;
    for (int j = lane; j < e; j += 32) {
      const float gz = to_f32(gt[m * ld + (size_t)h * e + j]);
      out[m * (size_t)(H * e) + (size_t)h * e + j] = from_f32<T>(vs[i * e8 + j] * r * (gz / (1.0f + expf(-gz))));
    }
  }
}

// Floats of scratch the chunked form needs for a step of M rows in B sequences.
LEB_API long long leb_retention_chunked_scratch(int M, int B, int H, int d, int e) {
  return ((long long)M / RC + B) * H * d * e;
}
LEB_API int leb_retention_chunked_supported(int d, int e) { return d >= 1 && e >= 1 && d <= 256 && e <= 256; }

LEB_API int leb_retention_chunked(void* out, const void* q, const void* k, const void* v, const void* g, int ld, int dtype,
                                  float* state, float* scratch, const float* decay, const float* inv_freq, int rot,
                                  float k_scale, float eps, const int* seq_slot, const int* seq_pos0,
                                  const int* seq_qstart, const int* seq_qlen, int M, int B, int H, int d, int e,
                                  cudaStream_t st) {
  if (M <= 0 || B <= 0) return 0;
  LEB_REQUIRE(dtype == LEB_F32 || dtype == LEB_BF16, "leb_retention_chunked: unknown dtype %d", dtype);
  LEB_REQUIRE(leb_retention_chunked_supported(d, e), "leb_retention_chunked: head sizes %d x %d outside 1..256", d, e);
  LEB_REQUIRE(rot >= 0 && rot <= d && rot % 2 == 0, "leb_retention_chunked: %d rotated dimensions do not fit %d", rot, d);
  LEB_REQUIRE(seq_qlen && scratch, "leb_retention_chunked: needs the sequences' row counts and scratch");
  LEB_REQUIRE(B <= 65535 && H <= 65535, "leb_retention_chunked: %d sequences, %d heads", B, H);
  const int d8 = (d + 7) & ~7, e8 = (e + 7) & ~7;
  const int chunks = M / RC + B;       // at least as many as the step has
  const size_t smem1 = (size_t)(RC * d8 + RC * e8 + RC) * sizeof(float);
  const size_t smem3 = (size_t)(2 * RC * d8 + RC * e8 + RC * (RC + 1) + RC + 1) * sizeof(float);
#define LEB_RC_ATTR(kern, bytes)                                                                              \
  if ((bytes) > 48 * 1024) {                                                                                  \
    cudaError_t er = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(bytes));   \
    if (er != cudaSuccess) return leb_fail("leb_retention_chunked: shared memory %zu: %s", (size_t)(bytes), cudaGetErrorString(er)); \
  }
  if (dtype == LEB_F32) {
    LEB_RC_ATTR(retention_chunk_state_kernel<float>, smem1);
    LEB_RC_ATTR(retention_chunk_out_kernel<float>, smem3);
    leb_launch(retention_chunk_state_kernel<float>, dim3(chunks, H), dim3(RCT), smem1, st, scratch, (const float*)q,
               (const float*)k, (const float*)v, ld, decay, inv_freq, rot, k_scale, seq_pos0, seq_qstart, seq_qlen, B, H, d, e);
  } else {
    LEB_RC_ATTR(retention_chunk_state_kernel<bf16>, smem1);
    LEB_RC_ATTR(retention_chunk_out_kernel<bf16>, smem3);
    leb_launch(retention_chunk_state_kernel<bf16>, dim3(chunks, H), dim3(RCT), smem1, st, scratch, (const bf16*)q,
               (const bf16*)k, (const bf16*)v, ld, decay, inv_freq, rot, k_scale, seq_pos0, seq_qstart, seq_qlen, B, H, d, e);
  }
  LEB_CHECK_LAUNCH("leb_retention_chunked states");
  leb_launch(retention_chunk_scan_kernel, dim3(ceil_div(d * e, 256), H, B), dim3(256), 0, st, scratch, state, decay,
             seq_slot, seq_qlen, B, H, d * e);
  LEB_CHECK_LAUNCH("leb_retention_chunked scan");
  if (dtype == LEB_F32)
    leb_launch(retention_chunk_out_kernel<float>, dim3(chunks, H), dim3(RCT), smem3, st, (float*)out, (const float*)scratch,
               (const float*)q, (const float*)k, (const float*)v, (const float*)g, ld, decay, inv_freq, rot, k_scale, eps,
               seq_pos0, seq_qstart, seq_qlen, B, H, d, e);
  else
    leb_launch(retention_chunk_out_kernel<bf16>, dim3(chunks, H), dim3(RCT), smem3, st, (bf16*)out, (const float*)scratch,
               (const bf16*)q, (const bf16*)k, (const bf16*)v, (const bf16*)g, ld, decay, inv_freq, rot, k_scale, eps,
               seq_pos0, seq_qstart, seq_qlen, B, H, d, e);
  LEB_CHECK_LAUNCH("leb_retention_chunked outputs");
#undef LEB_RC_ATTR
  return 0;
}
