// Latent attention on the tensor cores (bfloat16): the same arithmetic as latent_attention.cu's general
// kernel, for latents whose sizes fit the mma tiles (rank a multiple of 32 up to 512, rotated part a
// multiple of 16).
//
// A block of 8 warps owns one sequence, up to 64 query vectors (QT rows x HC heads; all heads read the
// same cached rows, so heads stack into the M dimension of the products) and one split of the key
// range.  Cached rows [c | k^r] come in tiles of BN = 64 (32 for latents beyond 256) through two shared-memory
// stages filled by asynchronous copies, the next tile travelling under the current one's products.  Per tile:
//   S = Q K^T        64 x BN over rank + rot     warp (m-tile of 16 vectors, half of the keys), mma.sync m16n8k16
//   softmax          float: four threads per vector, a quarter of the keys each; running maximum and sum in registers
//   O = O corr + P V 64 x rank over the BN keys  warp (32 vectors, a quarter of the latent), P as bfloat16,
//                    V = the first `rank` numbers of the same staged rows, read transposed by ldmatrix
// The accumulators of O (64 x rank floats, 128 registers a thread at rank 512) are why the latent is
// cut over four warps and a block is alone on its SM.  At the end the sink joins the denominator (or,
// with splits, maximum, sum and sums of c go to the partial buffer that latent_attention.cu merges).
#include "common.cuh"

#define LM_BM 64
#define LM_NEG (-1e30f)

__device__ __forceinline__ void lm_mma(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void lm_ldsm4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lm_ldsm4t(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lm_cp16(uint32_t dst, const void* src, int bytes) {   // bytes 16 or 0 (then zeros)
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void lm_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void lm_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }
__device__ __forceinline__ uint32_t lm_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// NT: n8-tiles of the latent a warp sums at most (rank <= 32 * NT).  BN: cached rows per tile, 64 where two
// stages of them fit shared memory beside the queries (rows of up to 512 numbers), else 32.
template <int NT, int BN>
__global__ void __launch_bounds__(256, 1)
latent_attention_mma_kernel(bf16* __restrict__ out, float* __restrict__ part, const bf16* __restrict__ qt,
                            const bf16* __restrict__ qr, const bf16* __restrict__ pool,
                            const int* __restrict__ block_table, int bt_width, const int* __restrict__ seq_slot,
                            const int* __restrict__ seq_pos0, const int* __restrict__ seq_qstart,
                            const int* __restrict__ seq_qlen, const float* __restrict__ sink, int M, int H,
                            int rank, int rot, int page_size, float scale, int QT, int HC, int n_splits) {
  extern __shared__ __align__(16) unsigned char lm_sm[];
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int hc = blockIdx.y;
  const int b = blockIdx.z / n_splits, split = blockIdx.z % n_splits;
  const int slot = seq_slot[b];
  const int qlen = seq_qlen[b];
  // the last rows of a prompt look back over the most keys: their blocks go first, the short ones fill the end
  const int row_lo = (gridDim.x - 1 - blockIdx.x) * QT;
  if (row_lo >= qlen) return;
  const int nrows = min(QT, qlen - row_lo);
  const int nheads = min(HC, H - hc * HC);
  const int q0 = seq_qstart[b];
  const int pos0 = seq_pos0[b];
  const int R = nrows * HC;                  // vectors r = i * HC + j in use (those with j >= nheads are idle)
  const int dk = rank + rot;
  const int LDK = dk + 8;                    // row stride in elements: an odd number of 16-byte pieces
  constexpr int LM_BN = BN;
  constexpr int LDP = BN + 8;
  constexpr int LDS = BN + 1;
  constexpr int KW = BN / 2;                 // keys of a warp's part of S
  const int ntu = rank / 32;                 // n8-tiles of the latent per warp

  bf16* q_s = reinterpret_cast<bf16*>(lm_sm);                      // [64][LDK]
  bf16* k_s = q_s + LM_BM * LDK;                                   // [2][32][LDK]
  float* s_s = reinterpret_cast<float*>(k_s + 2 * LM_BN * LDK);    // [64][BN + 1]
  bf16* p_s = reinterpret_cast<bf16*>(s_s + LM_BM * LDS);          // [64][LDP]
  float* c_s = reinterpret_cast<float*>(p_s + LM_BM * LDP);        // [64]

  if (slot < 0) {                            // a padding sequence: defined output, no cache access
    for (int r = warp; r < R; r += 8) {
      const int i = r / HC, j = r % HC;
      if (j >= nheads) continue;
      const int h = hc * HC + j;
      const size_t m = (size_t)q0 + row_lo + i;
      if (n_splits == 1) {
        for (int d = lane; d < rank; d += 32) out[((size_t)h * M + m) * rank + d] = __float2bfloat16_rn(0.f);
      } else {
        float* pp = part + ((m * H + h) * n_splits + split) * (size_t)(rank + 2);
        if (lane == 0) { pp[0] = LM_NEG; pp[1] = 0.f; }
        for (int d = lane; d < rank; d += 32) pp[2 + d] = 0.f;
      }
    }
    return;
  }

  // the query vectors [t_h | q_h^r], 16 bytes at a time; idle vectors are zeros
  const int cpr = dk / 8;                    // 16-byte pieces of a row
  for (int idx = tid; idx < LM_BM * cpr; idx += 256) {
    const int r = idx / cpr, c = idx - r * cpr;
    const int i = r / HC, j = r % HC;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < R && j < nheads) {
      const int h = hc * HC + j;
      const size_t m = (size_t)q0 + row_lo + i;
      const bf16* src = c * 8 < rank ? qt + ((size_t)h * M + m) * rank + c * 8
                                     : qr + (m * H + h) * (size_t)rot + (c * 8 - rank);
      v = *reinterpret_cast<const uint4*>(src);
    }
    *reinterpret_cast<uint4*>(q_s + (size_t)r * LDK + c * 8) = v;
  }
  for (int idx = tid; idx < LM_BM * LDP; idx += 256) p_s[idx] = __float2bfloat16_rn(0.f);
  if (tid < LM_BM) c_s[tid] = 1.f;

  const int kv_len = pos0 + qlen;
  const int pos_hi = pos0 + row_lo + nrows - 1;
  const int n_tiles = pos_hi / LM_BN + 1;
  const int per_split = (n_tiles + n_splits - 1) / n_splits;
  const int t_lo = split * per_split;
  const int t_hi = min(n_tiles, t_lo + per_split);

  auto load_tile = [&](int stage, int tile) {
    const int key0 = tile * LM_BN;
    const int page = block_table[(size_t)b * bt_width + key0 / page_size];
    const bf16* base = pool + ((size_t)(page < 0 ? 0 : page) * page_size + key0 % page_size) * dk;
    bf16* dst = k_s + (size_t)stage * LM_BN * LDK;
    for (int idx = tid; idx < LM_BN * cpr; idx += 256) {
      const int kk = idx / cpr, c = idx - kk * cpr;
      const bool live = page >= 0 && key0 + kk < kv_len;      // beyond the sequence the pool holds stale bits
      lm_cp16(lm_smem(dst + (size_t)kk * LDK + c * 8), live ? base + (size_t)kk * dk + c * 8 : pool, live ? 16 : 0);
    }
    lm_commit();
  };

  float o[2][NT][4];
#pragma unroll
  for (int a = 0; a < 2; a++)
#pragma unroll
    for (int n = 0; n < NT; n++)
#pragma unroll
      for (int e = 0; e < 4; e++) o[a][n][e] = 0.f;
  // softmax: four threads per query vector (vector tid / 4), each with a quarter of the tile's keys; the
  // running maximum and sum of the vector live in all four
  const int sm_r = tid >> 2, sm_q = tid & 3;
  float mx = LM_NEG, l = 0.f;

  const int g = lane >> 2, tg = lane & 3;
  // S: this warp's 16 vectors and half of the tile's keys;  O: this warp's 32 vectors and quarter of the latent
  const int s_mt = warp >> 1, s_kh = warp & 1;
  const int o_mh = warp >> 2, o_dq = warp & 3;
  const int dim0 = o_dq * 8 * ntu;
  const uint32_t q_addr = lm_smem(q_s + (size_t)(16 * s_mt + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + (lane >> 4) * 8);
  const uint32_t kb_off = (uint32_t)(((KW * s_kh + (lane & 7) + (lane >> 4) * 8) * LDK + ((lane >> 3) & 1) * 8) * 2);
  const uint32_t vb_off = (uint32_t)((((lane & 7) + ((lane >> 3) & 1) * 8) * LDK + dim0 + (lane >> 4) * 8) * 2);
  const uint32_t p_addr = lm_smem(p_s + (size_t)(32 * o_mh + (lane & 7) + ((lane >> 3) & 1) * 8) * LDP + (lane >> 4) * 8);

  if (t_lo < t_hi) load_tile(0, t_lo);
  for (int tile = t_lo; tile < t_hi; tile++) {
    const int stage = (tile - t_lo) & 1;
    lm_wait_all();
    __syncthreads();                         // the tile is there; everyone is done with the one before it
    if (tile + 1 < t_hi) load_tile(stage ^ 1, tile + 1);
    const int key0 = tile * LM_BN;
    const uint32_t k_base = lm_smem(k_s + (size_t)stage * LM_BN * LDK);

    // ---- S = Q K^T ----  Even and odd slices of the inner size sum in accumulators of their own, and a slice's
    // fragments are asked for before the products of the slice before it are issued: with two warps per
    // scheduler nothing else hides the way from shared memory or from one product to the next on its chain.
    if (16 * s_mt < R) {
      float s[2][KW / 8][4];
#pragma unroll
      for (int c = 0; c < 2; c++)
#pragma unroll
        for (int nt = 0; nt < KW / 8; nt++)
#pragma unroll
          for (int e = 0; e < 4; e++) s[c][nt][e] = 0.f;
      uint32_t a0[4], b0[KW / 16][4], a1[4], b1[KW / 16][4];
      lm_ldsm4(a0, q_addr);
#pragma unroll
      for (int np = 0; np < KW / 16; np++) lm_ldsm4(b0[np], k_base + kb_off + (uint32_t)(np * 16 * LDK * 2));
      for (int ks = 0; ks < dk; ks += 32) {
        const bool odd = ks + 16 < dk, more = ks + 32 < dk;
        if (odd) {
          lm_ldsm4(a1, q_addr + (ks + 16) * 2);
#pragma unroll
          for (int np = 0; np < KW / 16; np++) lm_ldsm4(b1[np], k_base + kb_off + (uint32_t)(np * 16 * LDK * 2) + (ks + 16) * 2);
        }
#pragma unroll
        for (int np = 0; np < KW / 16; np++) {
          lm_mma(s[0][2 * np], a0, b0[np][0], b0[np][1]);
          lm_mma(s[0][2 * np + 1], a0, b0[np][2], b0[np][3]);
        }
        if (more) {
          lm_ldsm4(a0, q_addr + (ks + 32) * 2);
#pragma unroll
          for (int np = 0; np < KW / 16; np++) lm_ldsm4(b0[np], k_base + kb_off + (uint32_t)(np * 16 * LDK * 2) + (ks + 32) * 2);
        }
        if (odd) {
#pragma unroll
          for (int np = 0; np < KW / 16; np++) {
            lm_mma(s[1][2 * np], a1, b1[np][0], b1[np][1]);
            lm_mma(s[1][2 * np + 1], a1, b1[np][2], b1[np][3]);
          }
        }
      }
#pragma unroll
      for (int half = 0; half < 2; half++) {
        const int r = 16 * s_mt + g + 8 * half;
        const int qpos = pos0 + row_lo + r / HC;
#pragma unroll
        for (int nt = 0; nt < KW / 8; nt++)
#pragma unroll
          for (int e = 0; e < 2; e++) {
            const int col = KW * s_kh + 8 * nt + 2 * tg + e;
            s_s[r * LDS + col] = key0 + col <= qpos ? (s[0][nt][2 * half + e] + s[1][nt][2 * half + e]) * scale : LM_NEG;
          }
      }
    }
    __syncthreads();

    // ---- softmax over the tile's keys: thread (vector, quarter) takes keys 8 q .. 8 q + 7 of every 32 (the
    // rows of S are 1 mod 32 words apart, so the 8 vectors x 4 quarters of a warp meet 32 different banks) ----
    {
      float sv[BN / 4];
      float tmax = LM_NEG;
#pragma unroll
      for (int c = 0; c < BN / 32; c++)
#pragma unroll
        for (int j = 0; j < 8; j++) {
          sv[8 * c + j] = sm_r < R ? s_s[sm_r * LDS + 32 * c + 8 * sm_q + j] : LM_NEG;
          tmax = fmaxf(tmax, sv[8 * c + j]);
        }
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
      const float mn = fmaxf(mx, tmax);
      float tsum = 0.f;
#pragma unroll
      for (int c = 0; c < BN / 32; c++) {
        uint32_t pk[4];
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          const float p0 = sv[8 * c + j] > 0.5f * LM_NEG ? expf(sv[8 * c + j] - mn) : 0.f;
          const float p1 = sv[8 * c + j + 1] > 0.5f * LM_NEG ? expf(sv[8 * c + j + 1] - mn) : 0.f;
          tsum += p0 + p1;
          __nv_bfloat162 two = __floats2bfloat162_rn(p0, p1);
          pk[j >> 1] = *reinterpret_cast<uint32_t*>(&two);
        }
        *reinterpret_cast<uint4*>(p_s + sm_r * LDP + 32 * c + 8 * sm_q) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      tsum += __shfl_xor_sync(0xffffffffu, tsum, 1);
      tsum += __shfl_xor_sync(0xffffffffu, tsum, 2);
      const float corr = expf(mx - mn);
      l = l * corr + tsum;
      mx = mn;
      if (sm_q == 0) c_s[sm_r] = corr;
    }
    __syncthreads();

    // ---- O = O corr + P V ----
#pragma unroll
    for (int mt = 0; mt < 2; mt++) {
      const int r0 = 32 * o_mh + 16 * mt;
      if (r0 >= R) break;
      const float ca = c_s[r0 + g], cb = c_s[r0 + g + 8];
      if (ca != 1.f || cb != 1.f) {          // once a vector's maximum has settled its sums stay as they are
#pragma unroll
        for (int n = 0; n < NT; n++) {
          o[mt][n][0] *= ca; o[mt][n][1] *= ca; o[mt][n][2] *= cb; o[mt][n][3] *= cb;
        }
      }
    }
    if (32 * o_mh < R) {
      const bool two = 32 * o_mh + 16 < R;
#pragma unroll
      for (int ks = 0; ks < BN / 16; ks++) {
        uint32_t a[2][4], bb[4], bn[4];
        lm_ldsm4(a[0], p_addr + ks * 32);
        lm_ldsm4(a[1], p_addr + 16 * LDP * 2 + ks * 32);
        const uint32_t v_addr = k_base + vb_off + (uint32_t)(ks * 16 * LDK * 2);
        lm_ldsm4t(bb, v_addr);
#pragma unroll
        for (int np = 0; np < NT / 2; np++) {
          if (np + 1 < NT / 2 && 2 * (np + 1) < ntu) lm_ldsm4t(bn, v_addr + (np + 1) * 32);
          if (2 * np < ntu) {
            lm_mma(o[0][2 * np], a[0], bb[0], bb[1]);
            if (2 * np + 1 < ntu) lm_mma(o[0][2 * np + 1], a[0], bb[2], bb[3]);
            if (two) {
              lm_mma(o[1][2 * np], a[1], bb[0], bb[1]);
              if (2 * np + 1 < ntu) lm_mma(o[1][2 * np + 1], a[1], bb[2], bb[3]);
            }
          }
#pragma unroll
          for (int e = 0; e < 4; e++) bb[e] = bn[e];
        }
      }
    }
  }
  __syncthreads();

  // ---- the end: the sink joins the denominator, or the split's partial sums go out ----
  if (sm_q == 0 && sm_r < R) {
    const int r = sm_r;
    const int i = r / HC, j = r % HC;
    if (j >= nheads) {
      c_s[r] = 0.f;
    } else {
      const int h = hc * HC + j;
      if (n_splits == 1) {
        const float sk = sink ? sink[h] : LM_NEG;
        const float mn = fmaxf(mx, sk);
        const float corr = expf(mx - mn);
        const float den = l * corr + (sink ? expf(sk - mn) : 0.f);
        c_s[r] = den > 0.f ? corr / den : 0.f;
      } else {
        const size_t m = (size_t)q0 + row_lo + i;
        float* pp = part + ((m * H + h) * n_splits + split) * (size_t)(rank + 2);
        pp[0] = mx;
        pp[1] = l;
        c_s[r] = 1.f;
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int mt = 0; mt < 2; mt++) {
#pragma unroll
    for (int half = 0; half < 2; half++) {
      const int r = 32 * o_mh + 16 * mt + g + 8 * half;
      if (r >= R) continue;
      const int i = r / HC, j = r % HC;
      if (j >= nheads) continue;
      const int h = hc * HC + j;
      const size_t m = (size_t)q0 + row_lo + i;
      const float f = c_s[r];
#pragma unroll
      for (int n = 0; n < NT; n++) {
        if (n >= ntu) break;
        const int d = dim0 + 8 * n + 2 * tg;
        const float v0 = o[mt][n][2 * half] * f, v1 = o[mt][n][2 * half + 1] * f;
        if (n_splits == 1) {
          *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)h * M + m) * rank + d) = __floats2bfloat162_rn(v0, v1);
        } else {
          float* pp = part + ((m * H + h) * n_splits + split) * (size_t)(rank + 2) + 2 + d;
          pp[0] = v0;
          pp[1] = v1;
        }
      }
    }
  }
}

// Whether the tensor-core kernel takes these sizes (bfloat16 only; the caller checks the type).
LEB_API int leb_latent_attention_mma_supported(int rank, int rot, int page_size) {
  return rank >= 32 && rank <= 512 && rank % 32 == 0 && rot >= 0 && rot <= 256 && rot % 16 == 0 && page_size % 64 == 0;
}

template <int NT, int BN>
static int launch_latent_mma(bf16* out, float* part, const bf16* qt, const bf16* qr, const bf16* pool,
                             const int* block_table, int bt_width, const int* seq_slot, const int* seq_pos0,
                             const int* seq_qstart, const int* seq_qlen, const float* sink, int M, int B, int H, int rank,
                             int rot, int page_size, float scale, int max_qlen, int n_splits, cudaStream_t st) {
  const int HC = H < LM_BM ? H : LM_BM;
  int QT = LM_BM / HC;
  if (QT > max_qlen) QT = max_qlen;
  const int dk = rank + rot;
  const size_t smem = (size_t)(LM_BM + 2 * BN) * (dk + 8) * 2 + (size_t)LM_BM * (BN + 1) * 4 + (size_t)LM_BM * (BN + 8) * 2 + LM_BM * 4;
  auto kern = latent_attention_mma_kernel<NT, BN>;
  static size_t smem_set = 0;
  if (smem > 48 * 1024 && smem > smem_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return leb_fail("leb_latent_attention_mma: shared memory %zu: %s", smem, cudaGetErrorString(e));
    smem_set = smem;
  }
  dim3 grid(ceil_div(max_qlen, QT), ceil_div(H, HC), B * n_splits);
  LEB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "leb_latent_attention_mma: grid too large (%u, %u)", grid.y, grid.z);
  leb_launch(kern, grid, dim3(256), smem, st, out, part, qt, qr, pool, block_table, bt_width, seq_slot, seq_pos0,
             seq_qstart, seq_qlen, sink, M, H, rank, rot, page_size, scale, QT, HC, n_splits);
  LEB_CHECK_LAUNCH("leb_latent_attention_mma");
  return 0;
}

// As leb_latent_attention for bfloat16 tensors with out rows exactly `rank` wide; with n_splits > 1 it
// leaves the partial sums in `part` and the caller runs the merge (leb_latent_merge).
LEB_API int leb_latent_attention_mma(void* out, float* part, const void* qt, const void* qr, const void* pool,
                                     const int* block_table, int bt_width, const int* seq_slot, const int* seq_pos0,
                                     const int* seq_qstart, const int* seq_qlen, const float* sink, int M, int B, int H,
                                     int rank, int rot, int page_size, float scale, int max_qlen, int n_splits,
                                     cudaStream_t st) {
  if (M <= 0 || B <= 0) return 0;
  LEB_REQUIRE(leb_latent_attention_mma_supported(rank, rot, page_size),
              "leb_latent_attention_mma: latent %d + %d with pages of %d is not a shape of this kernel", rank, rot, page_size);
  LEB_REQUIRE(n_splits >= 1 && (n_splits == 1 || (max_qlen == 1 && part)),
              "leb_latent_attention_mma: splits need single-row sequences and scratch");
  LEB_REQUIRE((((uintptr_t)qt | (uintptr_t)qr | (uintptr_t)pool) & 15) == 0, "leb_latent_attention_mma: operands must be 16-byte aligned");
  LebPlainLaunches plain(true);
#define LEB_LM(NT_, BN_)                                                                                                   \
  launch_latent_mma<NT_, BN_>((bf16*)out, part, (const bf16*)qt, (const bf16*)qr, (const bf16*)pool, block_table, bt_width, \
                              seq_slot, seq_pos0, seq_qstart, seq_qlen, sink, M, B, H, rank, rot, page_size, scale, max_qlen,  \
                              n_splits, st)
  if (rank <= 64) return LEB_LM(2, 64);
  if (rank <= 128) return LEB_LM(4, 64);
  if (rank <= 256) return LEB_LM(8, 64);
  return LEB_LM(16, 32);         // two stages of 64 rows of up to 768 numbers would not fit beside the queries
#undef LEB_LM
}
