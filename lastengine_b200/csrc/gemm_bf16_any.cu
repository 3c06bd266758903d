// bfloat16 product for operands the other kernels do not take: an inner size that is no multiple of 8, or
// rows that do not start on 16 bytes.  C (+)= A . W^T with float accumulation, 16 x 16 outputs per block,
// k in order in slices of 16 (a row's result does not depend on the other rows); with group_offsets the rows are
// grouped by expert as in the other grouped products.  Plain loads, CUDA cores:
// it is the way for odd sizes to run at all, not a fast path.
#include "common.cuh"

template <typename TC>
__global__ void __launch_bounds__(256) gemm_bf16_any_kernel(TC* __restrict__ C, const bf16* __restrict__ A,
                                                            const bf16* __restrict__ W, int M, int N, int K, int lda,
                                                            int ldc, int epilogue, const int* __restrict__ group_offsets,
                                                            size_t w_group_stride) {
  __shared__ float as[16][17], ws[16][17];
  pdl_trigger();
  pdl_wait();
  const int tx = threadIdx.x, ty = threadIdx.y;
  int row_begin = 0;
  if (group_offsets) {      // rows grouped by expert: group z owns rows [off[z], off[z+1]) and its own weights
    row_begin = group_offsets[blockIdx.z];
    M = group_offsets[blockIdx.z + 1];
    W += (size_t)blockIdx.z * w_group_stride;
    if (row_begin + (int)blockIdx.y * 16 >= M) return;
  }
  const int m = row_begin + blockIdx.y * 16 + ty, n = blockIdx.x * 16 + tx, wn = blockIdx.x * 16 + ty;
  float acc = 0.f;
  for (int k0 = 0; k0 < K; k0 += 16) {
    as[ty][tx] = (m < M && k0 + tx < K) ? to_f32(A[(size_t)m * lda + k0 + tx]) : 0.f;
    ws[ty][tx] = (wn < N && k0 + tx < K) ? to_f32(W[(size_t)wn * K + k0 + tx]) : 0.f;
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; kk++) acc += as[ty][kk] * ws[tx][kk];
    __syncthreads();
  }
  if (m < M && n < N) {
    TC* c = C + (size_t)m * ldc + n;
    *c = from_f32<TC>(epilogue == 1 ? to_f32(*c) + acc : acc);
  }
}

LEB_API int leb_gemm_bf16_any(void* C, int c_dtype, const void* A, const void* W, int M, int N, int K, int lda, int ldc,
                              int epilogue, const int* group_offsets, int n_groups, size_t w_group_stride, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  LEB_REQUIRE(epilogue == 0 || epilogue == 1, "leb_gemm_bf16_any: epilogue %d (store or add only)", epilogue);
  LEB_REQUIRE(epilogue != 1 || c_dtype == LEB_F32, "leb_gemm_bf16_any: adding needs a float C");
  const dim3 grid(ceil_div(N, 16), ceil_div(M, 16), group_offsets ? n_groups : 1), block(16, 16);
  LEB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "leb_gemm_bf16_any: %d rows or %d groups in one launch", M, n_groups);
  if (c_dtype == LEB_F32)
    leb_launch(gemm_bf16_any_kernel<float>, grid, block, 0, st, (float*)C, (const bf16*)A, (const bf16*)W, M, N, K, lda, ldc, epilogue, group_offsets, w_group_stride);
  else if (c_dtype == LEB_BF16)
    leb_launch(gemm_bf16_any_kernel<bf16>, grid, block, 0, st, (bf16*)C, (const bf16*)A, (const bf16*)W, M, N, K, lda, ldc, epilogue, group_offsets, w_group_stride);
  else
    return leb_fail("leb_gemm_bf16_any: unknown C dtype %d", c_dtype);
  LEB_CHECK_LAUNCH("leb_gemm_bf16_any");
  return 0;
}
