// Latent attention: every head's keys and values are linear images of one cached latent vector
// per position, plus one rotated key part that all heads share.
//
//   c_q = rmsnorm(W_dq h),  q_h = W_uq,h c_q = [q_h^n (dim) | q_h^r (rot)]      q_h^r rotated by position
//   [a | r] = W_dkv h,  c = rmsnorm(a) (rank),  k^r = rotate(r) (rot)              cached: [c | k^r]
//   k_h = W_uk,h c,  v_h = W_uv,h c
//   s_h(i, j) = scale (q_h^n . k_h(j) + q_h^r . k^r(j)),  j <= i
//   p = softmax over {s_h(i, j)} and one more logit sink_h that has no key and no value
//   o_h = sum_j p_j v_h(j)
//
// Only [c | k^r] is cached, one row of rank + rot numbers per position and layer, whatever the
// number of heads.  The kernels never form k_h or v_h: since q^n . (W_uk c) = (W_uk^T q^n) . c, a
// query is taken into the latent space once (t_h = W_uk,h^T q_h^n, a product grouped by head),
// attention runs with the one cached row as key ([c | k^r] against [t_h | q_h^r]) and its first
// `rank` numbers as value, and the result u_h = sum_j p_j c(j) goes through W_uv,h afterwards
// (again a product grouped by head).  All heads of a row share every key they read.
//
// Kernels here: the preparation of a step's rows (both norms, the rotation of k^r, the cache
// write), the split of q into its unrotated part (head-major, for the grouped product) and its
// rotated part, the attention itself with its merge of key-range splits, and the turn of a
// head-major result back to rows.  Norms, angles, sine and cosine, scores, softmax and the value
// sums are float; sinf/cosf are the full-range versions.
#include "common.cuh"

// Rotation of the first `rot_dims` of `n` numbers, pairs (2i, 2i + 1): (u, v) -> (u cos a - v sin a,
// v cos a + u sin a), a = pos * inv_freq[i]; the rest passes unchanged.
__device__ __forceinline__ float rot_pair(float u, float v, float c, float s, int odd) {
  return odd ? v * c + u * s : u * c - v * s;
}

// One block per row.  in [M, ld_in]: columns [0, q_rank) the query latent before its norm, then
// (own_kv) `rank` columns of the key/value latent before its norm and `rot` columns of the shared
// key part before its rotation.  Leaves cq [M, q_rank] = rmsnorm(.) * wq and, for rows of live
// sequences, the cache row [c | k^r] at the row's position.
template <typename T, typename CT>
__global__ void __launch_bounds__(256)
latent_prep_kernel(T* __restrict__ cq, const T* __restrict__ in, int ld_in, CT* __restrict__ pool,
                   const int* __restrict__ block_table, int bt_width, const int* __restrict__ row_seq,
                   const int* __restrict__ row_pos, const int* __restrict__ seq_slot,
                   const float* __restrict__ wq, const float* __restrict__ wkv, float eps,
                   const float* __restrict__ inv_freq, int rot_dims, int q_rank, int rank, int rot,
                   int page_size) {
  __shared__ float red[33];
  pdl_wait();
  const int m = blockIdx.x;
  const T* row = in + (size_t)m * ld_in;
  float ss = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
    const float v = to_f32(row[i]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  float r = 1.0f / sqrtf(ss / (float)q_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    cq[(size_t)m * q_rank + i] = from_f32<T>(to_f32(row[i]) * r * wq[i]);
  if (!pool) return;
  const int b = row_seq[m], pos = row_pos[m];
  const T* lat = row + q_rank;
  ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_f32(lat[i]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  if (seq_slot[b] < 0) return;      // a padding sequence touches no cache
  const int page = block_table[(size_t)b * bt_width + pos / page_size];
  if (page < 0) return;
  r = 1.0f / sqrtf(ss / (float)rank + eps);
  CT* dst = pool + ((size_t)page * page_size + pos % page_size) * (size_t)(rank + rot);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f32<CT>(to_f32(lat[i]) * r * wkv[i]);
  const T* kr = lat + rank;
  for (int i = threadIdx.x; i < rot; i += blockDim.x) {
    float v = to_f32(kr[i]);
    if (i < rot_dims) {
      const float a = (float)pos * inv_freq[i >> 1];
      v = rot_pair(to_f32(kr[i & ~1]), to_f32(kr[i | 1]), cosf(a), sinf(a), i & 1);
    }
    dst[rank + i] = from_f32<CT>(v);
  }
}

// q [M, H * (dim + rot)] -> qn [H, M, dim_p] (the unrotated parts, head-major, zeros from dim to
// dim_p) and qr [M, H, rot] (the rotated parts).  One block per row.
template <typename T>
__global__ void __launch_bounds__(256)
latent_q_split_kernel(T* __restrict__ qn, T* __restrict__ qr, const T* __restrict__ q,
                      const int* __restrict__ row_pos, const float* __restrict__ inv_freq, int rot_dims,
                      int M, int H, int dim, int dim_p, int rot) {
  pdl_wait();
  const int m = blockIdx.x;
  const int hw = dim + rot;
  const T* row = q + (size_t)m * H * hw;
  constexpr int PER = 16 / (int)sizeof(T);          // elements of a 16-byte piece
  if (dim_p == dim && dim % PER == 0 && hw % PER == 0 && (((uintptr_t)q | (uintptr_t)qn) & 15) == 0) {
    const int pieces = dim / PER;
    for (int i = threadIdx.x; i < H * pieces; i += blockDim.x) {
      const int h = i / pieces, c = i - h * pieces;
      reinterpret_cast<uint4*>(qn + ((size_t)h * M + m) * dim)[c] = reinterpret_cast<const uint4*>(row + h * hw)[c];
    }
  } else {
    for (int i = threadIdx.x; i < H * dim_p; i += blockDim.x) {
      const int h = i / dim_p, d = i - h * dim_p;
      qn[((size_t)h * M + m) * dim_p + d] = d < dim ? row[h * hw + d] : from_f32<T>(0.f);
    }
  }
  const float pos = (float)row_pos[m];
  if (rot % 2 == 0) {       // a thread per pair: one sine and cosine for both numbers
    const int hp = rot / 2;
    for (int i = threadIdx.x; i < H * hp; i += blockDim.x) {
      const int h = i / hp, t = i - h * hp;
      const T* r = row + h * hw + dim + 2 * t;
      float u = to_f32(r[0]), v = to_f32(r[1]);
      if (2 * t < rot_dims) {
        const float a = pos * inv_freq[t];
        const float c = cosf(a), sn = sinf(a);
        const float u2 = u * c - v * sn;
        v = v * c + u * sn;
        u = u2;
      }
      T* o = qr + ((size_t)m * H + h) * rot + 2 * t;
      o[0] = from_f32<T>(u);
      o[1] = from_f32<T>(v);
    }
    return;
  }
  for (int i = threadIdx.x; i < H * rot; i += blockDim.x) {
    const int h = i / rot, d = i - h * rot;
    const T* r = row + h * hw + dim;
    float v = to_f32(r[d]);
    if (d < rot_dims) {
      const float a = pos * inv_freq[d >> 1];
      v = rot_pair(to_f32(r[d & ~1]), to_f32(r[d | 1]), cosf(a), sinf(a), d & 1);
    }
    qr[(size_t)m * H * rot + i] = from_f32<T>(v);
  }
}

// in [H, M, w] -> out [M, H * w], one piece per thread: an element, or 16 bytes where the rows allow it
template <typename P>
__global__ void heads_to_rows_kernel(P* __restrict__ out, const P* __restrict__ in, int M, int H, int w) {
  pdl_wait();
  const size_t total = (size_t)M * H * w;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t m = i / ((size_t)H * w);
  const int r = (int)(i - m * H * w);
  const int h = r / w, d = r - h * w;
  out[i] = in[((size_t)h * M + m) * w + d];
}

// ---------------------------------------------------------------------------------------------
// The attention.  Block = 4 warps: one sequence, a chunk of HC <= 8 heads, QT rows (QT * HC <= 32
// query vectors), one split of the key range.  Per tile of 32 cached rows, staged once as float
// for all of the block's query vectors: lane = key for the scores, lane = dimension for the sums
// of c.  A query vector is [t_h (rank) | q_h^r (rot)].
#define LAT_WARPS 4
#define LAT_RPW 8
#define LAT_NEG (-1e30f)

template <typename T, typename CT, int HDL>      // rank <= 32 * HDL
__global__ void __launch_bounds__(32 * LAT_WARPS)
latent_attention_kernel(T* __restrict__ out, int ld_out, float* __restrict__ part, const T* __restrict__ qt,
                        const T* __restrict__ qr, const CT* __restrict__ pool,
                        const int* __restrict__ block_table, int bt_width, const int* __restrict__ seq_slot,
                        const int* __restrict__ seq_pos0, const int* __restrict__ seq_qstart,
                        const int* __restrict__ seq_qlen, const float* __restrict__ sink, int M, int H,
                        int rank, int rot, int page_size, float scale, int QT, int HC, int n_splits) {
  extern __shared__ float sm[];
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int hc = blockIdx.y;
  const int b = blockIdx.z / n_splits, split = blockIdx.z % n_splits;
  const int slot = seq_slot[b];
  const int qlen = seq_qlen[b];
  const int row_lo = blockIdx.x * QT;
  if (row_lo >= qlen) return;
  const int nrows = min(QT, qlen - row_lo);
  const int nheads = min(HC, H - hc * HC);
  const int q0 = seq_qstart[b];
  const int pos0 = seq_pos0[b];
  const int R = QT * HC;
  const int dk = rank + rot;
  const int KS = dk + 1;           // lanes read different staged rows at the same column

  float* q_s = sm;                 // [R][dk]
  float* k_s = q_s + R * dk;       // [32][dk + 1]
  float* p_s = k_s + 32 * KS;      // [LAT_WARPS][32]

  if (slot < 0) {                  // a padding sequence: defined output, no cache access
    for (int r = warp; r < R; r += LAT_WARPS) {
      const int i = r / HC, j = r % HC;
      if (i >= nrows || j >= nheads) continue;
      const int h = hc * HC + j;
      const size_t m = (size_t)q0 + row_lo + i;
      if (n_splits == 1) {
        for (int d = lane; d < ld_out; d += 32) out[((size_t)h * M + m) * ld_out + d] = from_f32<T>(0.f);
      } else {
        float* pp = part + ((m * H + h) * n_splits + split) * (size_t)(rank + 2);
        if (lane == 0) { pp[0] = LAT_NEG; pp[1] = 0.f; }
        for (int d = lane; d < rank; d += 32) pp[2 + d] = 0.f;
      }
    }
    return;
  }

  for (int idx = threadIdx.x; idx < R * dk; idx += blockDim.x) {
    const int r = idx / dk, d = idx - r * dk;
    const int i = r / HC, j = r % HC;
    float v = 0.f;
    if (i < nrows && j < nheads) {
      const int h = hc * HC + j;
      const size_t m = (size_t)q0 + row_lo + i;
      v = d < rank ? to_f32(qt[((size_t)h * M + m) * rank + d]) : to_f32(qr[(m * H + h) * rot + (d - rank)]);
    }
    q_s[idx] = v;
  }

  const int kv_len = pos0 + qlen;
  const int pos_hi = pos0 + row_lo + nrows - 1;
  const int n_tiles = pos_hi / 32 + 1;
  const int per_split = (n_tiles + n_splits - 1) / n_splits;
  const int t_lo = split * per_split;
  const int t_hi = min(n_tiles, t_lo + per_split);

  float mx[LAT_RPW], l[LAT_RPW], acc[LAT_RPW][HDL];
#pragma unroll
  for (int ri = 0; ri < LAT_RPW; ri++) {
    mx[ri] = LAT_NEG;
    l[ri] = 0.f;
#pragma unroll
    for (int jj = 0; jj < HDL; jj++) acc[ri][jj] = 0.f;
  }

  for (int tile = t_lo; tile < t_hi; tile++) {
    const int key0 = tile * 32;
    const int page = block_table[(size_t)b * bt_width + key0 / page_size];
    const size_t base = ((size_t)(page < 0 ? 0 : page) * page_size + key0 % page_size) * dk;
    __syncthreads();               // the previous tile has been consumed (and q_s is written, first time round)
    for (int idx = threadIdx.x; idx < 32 * dk; idx += blockDim.x) {
      const int kk = idx / dk, d = idx - kk * dk;
      float kv = 0.f;
      if (page >= 0 && key0 + kk < kv_len) kv = to_f32(pool[base + idx]);   // beyond the sequence the pool holds stale bits
      k_s[kk * KS + d] = kv;
    }
    __syncthreads();
#pragma unroll
    for (int ri = 0; ri < LAT_RPW; ri++) {
      const int r = warp + ri * LAT_WARPS;
      if (r >= R) break;
      const int i = r / HC, j = r % HC;
      if (i >= nrows || j >= nheads) continue;
      const int qpos = pos0 + row_lo + i;
      if (key0 > qpos) continue;   // the whole tile lies after this row
      const float* qv = q_s + r * dk;
      const float* kr = k_s + lane * KS;
      float s = 0.f;
      for (int d = 0; d < dk; d++) s += qv[d] * kr[d];
      s *= scale;
      const bool valid = key0 + lane <= qpos;
      s = valid ? s : LAT_NEG;
      const float mn = fmaxf(mx[ri], warp_max(s));
      const float p = valid ? expf(s - mn) : 0.f;
      const float corr = expf(mx[ri] - mn);
      l[ri] = l[ri] * corr + warp_sum(p);
      mx[ri] = mn;
      p_s[warp * 32 + lane] = p;
      __syncwarp();
#pragma unroll
      for (int jj = 0; jj < HDL; jj++) {
        const int d = lane + 32 * jj;
        if (d < rank) {
          float a = 0.f;
#pragma unroll 8
          for (int kk = 0; kk < 32; kk++) a += p_s[warp * 32 + kk] * k_s[kk * KS + d];
          acc[ri][jj] = acc[ri][jj] * corr + a;
        }
      }
      __syncwarp();
    }
  }

#pragma unroll
  for (int ri = 0; ri < LAT_RPW; ri++) {
    const int r = warp + ri * LAT_WARPS;
    if (r >= R) break;
    const int i = r / HC, j = r % HC;
    if (i >= nrows || j >= nheads) continue;
    const int h = hc * HC + j;
    const size_t m = (size_t)q0 + row_lo + i;
    if (n_splits == 1) {
      // the sink joins the denominator: one more logit, not scaled, without a value
      const float sk = sink ? sink[h] : LAT_NEG;
      const float mn = fmaxf(mx[ri], sk);
      const float corr = expf(mx[ri] - mn);
      const float den = l[ri] * corr + (sink ? expf(sk - mn) : 0.f);
      const float inv = den > 0.f ? corr / den : 0.f;
      T* o = out + ((size_t)h * M + m) * ld_out;
#pragma unroll
      for (int jj = 0; jj < HDL; jj++) {
        const int d = lane + 32 * jj;
        if (d < rank) o[d] = from_f32<T>(acc[ri][jj] * inv);
      }
      for (int d = rank + lane; d < ld_out; d += 32) o[d] = from_f32<T>(0.f);
    } else {
      float* pp = part + ((m * H + h) * n_splits + split) * (size_t)(rank + 2);
      if (lane == 0) { pp[0] = mx[ri]; pp[1] = l[ri]; }
#pragma unroll
      for (int jj = 0; jj < HDL; jj++) {
        const int d = lane + 32 * jj;
        if (d < rank) pp[2 + d] = acc[ri][jj];
      }
    }
  }
}

// Merge of the key-range splits of one (row, head), with the sink as one more term of the
// denominator: out = sum_s acc_s e^(m_s - m) / (sum_s l_s e^(m_s - m) + e^(sink - m)).
template <typename T>
__global__ void latent_merge_kernel(T* __restrict__ out, int ld_out, const float* __restrict__ part,
                                    const float* __restrict__ sink, int M, int H, int rank, int n_splits) {
  pdl_wait();
  const size_t m = blockIdx.x;
  const int h = blockIdx.y;
  const size_t step = rank + 2;
  const float* pp = part + ((m * H + h) * n_splits) * step;
  float mn = sink ? sink[h] : LAT_NEG;
  for (int s = 0; s < n_splits; s++) mn = fmaxf(mn, pp[s * step]);
  float den = sink ? expf(sink[h] - mn) : 0.f;
  for (int s = 0; s < n_splits; s++) den += pp[s * step + 1] * expf(pp[s * step] - mn);
  const float inv = den > 0.f ? 1.0f / den : 0.f;
  T* o = out + ((size_t)h * M + m) * ld_out;
  for (int d = threadIdx.x; d < ld_out; d += blockDim.x) {
    float a = 0.f;
    if (d < rank)
      for (int s = 0; s < n_splits; s++) a += pp[s * step + 2 + d] * expf(pp[s * step] - mn);
    o[d] = from_f32<T>(a * inv);
  }
}

// ---------------------------------------------------------------------------------------------
LEB_API int leb_latent_prep(void* cq, const void* in, int ld_in, int dtype, void* pool, const int* block_table,
                            int bt_width, const int* row_seq, const int* row_pos, const int* seq_slot,
                            const float* wq, const float* wkv, float eps, const float* inv_freq, int rot_dims,
                            int M, int q_rank, int rank, int rot, int page_size, cudaStream_t st) {
  if (M <= 0) return 0;
  LEB_REQUIRE(q_rank >= 1 && wq, "leb_latent_prep: the query latent needs a width and a norm weight");
  LEB_REQUIRE(!pool || (rank >= 1 && rot >= 0 && wkv && block_table && row_seq && row_pos && seq_slot),
              "leb_latent_prep: a cache write needs the latent's sizes, its norm weight and the step's tables");
  LEB_REQUIRE(rot_dims >= 0 && rot_dims <= rot && rot_dims % 2 == 0 && (rot_dims == 0 || inv_freq),
              "leb_latent_prep: %d rotated dimensions of %d", rot_dims, rot);
  LebPlainLaunches plain(true);
  if (dtype == LEB_F32)
    leb_launch(latent_prep_kernel<float, float>, dim3(M), dim3(128), 0, st, (float*)cq, (const float*)in, ld_in,
               (float*)pool, block_table, bt_width, row_seq, row_pos, seq_slot, wq, wkv, eps, inv_freq, rot_dims,
               q_rank, rank, rot, page_size);
  else if (dtype == LEB_BF16)
    leb_launch(latent_prep_kernel<bf16, bf16>, dim3(M), dim3(128), 0, st, (bf16*)cq, (const bf16*)in, ld_in,
               (bf16*)pool, block_table, bt_width, row_seq, row_pos, seq_slot, wq, wkv, eps, inv_freq, rot_dims,
               q_rank, rank, rot, page_size);
  else
    return leb_fail("leb_latent_prep: unknown dtype %d", dtype);
  LEB_CHECK_LAUNCH("leb_latent_prep");
  return 0;
}

LEB_API int leb_latent_q_split(void* qn, void* qr, const void* q, int dtype, const int* row_pos,
                               const float* inv_freq, int rot_dims, int M, int H, int dim, int dim_p, int rot,
                               cudaStream_t st) {
  if (M <= 0) return 0;
  LEB_REQUIRE(H >= 1 && dim >= 1 && dim_p >= dim && rot >= 0, "leb_latent_q_split: sizes out of range");
  LEB_REQUIRE(rot_dims >= 0 && rot_dims <= rot && rot_dims % 2 == 0 && (rot_dims == 0 || inv_freq),
              "leb_latent_q_split: %d rotated dimensions of %d", rot_dims, rot);
  LebPlainLaunches plain(true);
  if (dtype == LEB_F32)
    leb_launch(latent_q_split_kernel<float>, dim3(M), dim3(256), 0, st, (float*)qn, (float*)qr, (const float*)q,
               row_pos, inv_freq, rot_dims, M, H, dim, dim_p, rot);
  else if (dtype == LEB_BF16)
    leb_launch(latent_q_split_kernel<bf16>, dim3(M), dim3(256), 0, st, (bf16*)qn, (bf16*)qr, (const bf16*)q, row_pos,
               inv_freq, rot_dims, M, H, dim, dim_p, rot);
  else
    return leb_fail("leb_latent_q_split: unknown dtype %d", dtype);
  LEB_CHECK_LAUNCH("leb_latent_q_split");
  return 0;
}

LEB_API int leb_heads_to_rows(void* out, const void* in, int dtype, int M, int H, int w, cudaStream_t st) {
  if ((size_t)M * H * w == 0) return 0;
  LEB_REQUIRE(dtype == LEB_F32 || dtype == LEB_BF16, "leb_heads_to_rows: unknown dtype %d", dtype);
  LebPlainLaunches plain(true);
  const int per16 = dtype == LEB_F32 ? 4 : 8;      // elements of a 16-byte piece
  if (w % per16 == 0 && (((uintptr_t)out | (uintptr_t)in) & 15) == 0) {
    const size_t total = (size_t)M * H * (w / per16);
    leb_launch(heads_to_rows_kernel<uint4>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, (uint4*)out,
               (const uint4*)in, M, H, w / per16);
  } else {
    const size_t total = (size_t)M * H * w;
    const dim3 grid((unsigned)((total + 255) / 256)), block(256);
    if (dtype == LEB_F32) leb_launch(heads_to_rows_kernel<float>, grid, block, 0, st, (float*)out, (const float*)in, M, H, w);
    else leb_launch(heads_to_rows_kernel<bf16>, grid, block, 0, st, (bf16*)out, (const bf16*)in, M, H, w);
  }
  LEB_CHECK_LAUNCH("leb_heads_to_rows");
  return 0;
}

template <typename T, int HDL>
static int launch_latent(void* out, int ld_out, float* part, const void* qt, const void* qr, const void* pool,
                         const int* block_table, int bt_width, const int* seq_slot, const int* seq_pos0,
                         const int* seq_qstart, const int* seq_qlen, const float* sink, int M, int B, int H, int rank,
                         int rot, int page_size, float scale, int max_qlen, int n_splits, cudaStream_t st) {
  const int HC = H < 8 ? H : 8;
  int QT = 32 / HC;
  if (QT > max_qlen) QT = max_qlen;
  const int R = QT * HC;
  const int dk = rank + rot;
  const size_t smem = ((size_t)R * dk + 32 * (dk + 1) + LAT_WARPS * 32) * sizeof(float);
  auto kern = latent_attention_kernel<T, T, HDL>;
  static size_t smem_set = 0;
  if (smem > 48 * 1024 && smem > smem_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return leb_fail("leb_latent_attention: shared memory %zu: %s", smem, cudaGetErrorString(e));
    smem_set = smem;
  }
  dim3 grid(ceil_div(max_qlen, QT), ceil_div(H, HC), B * n_splits);
  LEB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "leb_latent_attention: grid too large (%u, %u)", grid.y, grid.z);
  leb_launch(kern, grid, dim3(32 * LAT_WARPS), smem, st, (T*)out, ld_out, part, (const T*)qt, (const T*)qr,
             (const T*)pool, block_table, bt_width, seq_slot, seq_pos0, seq_qstart, seq_qlen, sink, M, H, rank, rot,
             page_size, scale, QT, HC, n_splits);
  LEB_CHECK_LAUNCH("leb_latent_attention");
  return 0;
}

// The tensor-core kernel for bfloat16 (latent_attention_mma.cu) and its switch (on by default; off for comparisons).
extern "C" int leb_latent_attention_mma_supported(int rank, int rot, int page_size);
extern "C" int leb_latent_attention_mma(void* out, float* part, const void* qt, const void* qr, const void* pool,
                                        const int* block_table, int bt_width, const int* seq_slot, const int* seq_pos0,
                                        const int* seq_qstart, const int* seq_qlen, const float* sink, int M, int B, int H,
                                        int rank, int rot, int page_size, float scale, int max_qlen, int n_splits,
                                        cudaStream_t st);
static int g_latent_mma = 1;
LEB_API void leb_set_latent_mma(int on) { g_latent_mma = on ? 1 : 0; }

// qt [H, M, rank] (queries taken into the latent space), qr [M, H, rot] (rotated parts), pool
// [page][page_size][rank + rot], sink [H] float or null; out [H, M, ld_out] (ld_out >= rank, the
// rest zeros).  part: float scratch of M*H*n_splits*(rank+2), used when n_splits > 1 (then every
// sequence brings one row).
LEB_API int leb_latent_attention(void* out, int ld_out, float* part, const void* qt, const void* qr, const void* pool,
                                 int dtype, const int* block_table, int bt_width, const int* seq_slot,
                                 const int* seq_pos0, const int* seq_qstart, const int* seq_qlen, const float* sink,
                                 int M, int B, int H, int rank, int rot, int page_size, float scale, int max_qlen,
                                 int n_splits, cudaStream_t st) {
  if (M <= 0 || B <= 0) return 0;
  LEB_REQUIRE(rank >= 1 && rank <= 512, "leb_latent_attention: latent size %d outside 1..512", rank);
  LEB_REQUIRE(rot >= 0 && rot <= 256, "leb_latent_attention: %d rotated dimensions outside 0..256", rot);
  LEB_REQUIRE(ld_out >= rank, "leb_latent_attention: result rows of %d for a latent of %d", ld_out, rank);
  LEB_REQUIRE(page_size % 32 == 0, "leb_latent_attention: page size %d is not a multiple of 32", page_size);
  LEB_REQUIRE(n_splits >= 1 && (n_splits == 1 || (max_qlen == 1 && part)),
              "leb_latent_attention: splits need single-row sequences and scratch");
  LebPlainLaunches plain(true);
  int rc;
  const bool mma = g_latent_mma && dtype == LEB_BF16 && ld_out == rank && leb_latent_attention_mma_supported(rank, rot, page_size) &&
                   (((uintptr_t)qt | (uintptr_t)qr | (uintptr_t)pool) & 15) == 0;
#define LEB_LAT(T, L)                                                                                              \
  launch_latent<T, L>(out, ld_out, part, qt, qr, pool, block_table, bt_width, seq_slot, seq_pos0, seq_qstart, seq_qlen, \
                      sink, M, B, H, rank, rot, page_size, scale, max_qlen, n_splits, st)
#define LEB_LAT_T(T) \
  (rank <= 32 ? LEB_LAT(T, 1) : rank <= 64 ? LEB_LAT(T, 2) : rank <= 128 ? LEB_LAT(T, 4) : rank <= 256 ? LEB_LAT(T, 8) : LEB_LAT(T, 16))
  if (mma)
    rc = leb_latent_attention_mma(out, part, qt, qr, pool, block_table, bt_width, seq_slot, seq_pos0, seq_qstart, seq_qlen,
                                  sink, M, B, H, rank, rot, page_size, scale, max_qlen, n_splits, st);
  else if (dtype == LEB_F32) rc = LEB_LAT_T(float);
  else if (dtype == LEB_BF16) rc = LEB_LAT_T(bf16);
  else return leb_fail("leb_latent_attention: unknown dtype %d", dtype);
#undef LEB_LAT_T
#undef LEB_LAT
  if (rc) return rc;
  if (n_splits > 1) {
    dim3 grid(M, H);
    if (dtype == LEB_F32)
      leb_launch(latent_merge_kernel<float>, grid, dim3(128), 0, st, (float*)out, ld_out, part, sink, M, H, rank, n_splits);
    else
      leb_launch(latent_merge_kernel<bf16>, grid, dim3(128), 0, st, (bf16*)out, ld_out, part, sink, M, H, rank, n_splits);
    LEB_CHECK_LAUNCH("leb_latent_attention merge");
  }
  return 0;
}
