// Per-head matrix products: out[t, h, :] = W[h] x[t, h, :] for every token t and head h, with
// W [H, N, K] dense and x / out addressed through a token stride and a head stride (so a slice of
// each head's columns can be read or written in place).  Accumulation is fp32 on the FMA pipes,
// one accumulator per output taking its K products in ascending k, so a token's result does not
// depend on how many tokens the step has (as in gemm_f32.cu); operands and results are fp32 or
// bfloat16.  Used where a product is block-diagonal over heads (moving queries into a latent space
// and attended latents out of it).
#include "common.cuh"

template <typename T, int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
head_gemm_kernel(const T* __restrict__ X, long xs_t, long xs_h, const T* __restrict__ W, T* __restrict__ C,
                 long os_t, long os_h, int M, int N, int K) {
  constexpr int BK = 16;
  constexpr int THREADS = (BM / TM) * (BN / TN);
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int h = blockIdx.z;
  const T* Xh = X + (long)h * xs_h;
  const T* Wh = W + (long)h * N * K;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int e = tid; e < BM * BK; e += THREADS) {
      const int r = e / BK, c = e % BK;
      const int gm = m0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? to_f32(Xh[(long)gm * xs_t + gk]) : 0.f;
    }
    for (int e = tid; e < BN * BK; e += THREADS) {
      const int r = e / BK, c = e % BK;
      const int gn = n0 + r, gk = k0 + c;
      Ws[c][r] = (gn < N && gk < K) ? to_f32(Wh[(long)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  T* Ch = C + (long)h * os_h;
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn < N) Ch[(long)gm * os_t + gn] = from_f32<T>(acc[i][j]);
    }
  }
}

// A handful of tokens (M <= 16) in bfloat16: the product is a stream of the heads' weights.  A block
// owns one head and 32 of its output rows; the tokens' rows of that head wait in shared memory as
// fp32; each warp streams four weight rows side by side, 16 bytes per lane, row and step, and the lanes' partial sums
// meet in a shuffle tree.  K is a multiple of 8 and weight rows are 16-byte aligned.
constexpr int HEAD_SMALL_M = 16;
__global__ void __launch_bounds__(256)
head_gemm_small_kernel(const bf16* __restrict__ X, long xs_t, long xs_h, const bf16* __restrict__ W,
                       bf16* __restrict__ C, long os_t, long os_h, int M, int N, int K) {
  extern __shared__ float xs[];  // [M][K]
  const int h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bf16* Xh = X + (long)h * xs_h;
  for (int i = threadIdx.x; i < M * K; i += 256) {
    const int t = i / K, k = i - t * K;
    xs[i] = to_f32(Xh[(long)t * xs_t + k]);
  }
  __syncthreads();
  const bf16* Wh = W + (long)h * N * K;
  const int n0 = blockIdx.x * 32 + warp * 4;  // this warp's four rows, streamed side by side
  float acc[4][HEAD_SMALL_M];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int t = 0; t < HEAD_SMALL_M; ++t) acc[r][t] = 0.f;
  for (int k = lane * 8; k < K; k += 256) {
    float w[4][8];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      if (n0 + r < N) {
        load8(Wh + (long)(n0 + r) * K + k, w[r]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) w[r][e] = 0.f;
      }
    }
#pragma unroll
    for (int t = 0; t < HEAD_SMALL_M; ++t) {
      if (t < M) {
        float x[8];
        load8(xs + t * K + k, x);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[r][t] = fmaf(w[r][e], x[e], acc[r][t]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    if (n0 + r >= N) continue;
#pragma unroll
    for (int t = 0; t < HEAD_SMALL_M; ++t) {
      if (t < M) {
        const float v = warp_sum(acc[r][t]);
        if (lane == 0) C[(long)t * os_t + (long)h * os_h + n0 + r] = from_f32<bf16>(v);
      }
    }
  }
}

template <typename T>
static int launch_head_gemm(const void* x, long xs_t, long xs_h, const void* w, void* out, long os_t, long os_h, int M,
                            int H, int N, int K, cudaStream_t stream) {
  if (M > 64) {
    dim3 grid((N + 127) / 128, (M + 127) / 128, H);
    if (grid.y > 65535) return Q3_ERR_UNSUPPORTED;
    head_gemm_kernel<T, 128, 128, 8, 8><<<grid, 256, 0, stream>>>((const T*)x, xs_t, xs_h, (const T*)w, (T*)out, os_t,
                                                                  os_h, M, N, K);
  } else {
    dim3 grid((N + 63) / 64, (M + 31) / 32, H);
    head_gemm_kernel<T, 32, 64, 2, 4><<<grid, 256, 0, stream>>>((const T*)x, xs_t, xs_h, (const T*)w, (T*)out, os_t,
                                                                os_h, M, N, K);
  }
  return q3_launch_status();
}

// x: (t, h, k) at x + t*xs_t + h*xs_h + k; w: [H, N, K]; out: (t, h, n) at out + t*os_t + h*os_h + n.
Q3_EXPORT int q3_head_linear(int dtype, const void* x, long xs_t, long xs_h, const void* w, void* out, long os_t,
                             long os_h, int M, int H, int N, int K, cudaStream_t stream) {
  if (!x || !w || !out || H < 1 || N < 1 || K < 1) return Q3_ERR_ARGUMENT;
  if (H > 65535) return Q3_ERR_UNSUPPORTED;
  if (M == 0) return Q3_OK;
  if (dtype == Q3_DTYPE_BF16 && M <= HEAD_SMALL_M && K % 8 == 0 && (size_t)M * K * sizeof(float) <= 96 * 1024 &&
      (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
    const size_t smem = (size_t)M * K * sizeof(float);
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(head_gemm_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    head_gemm_small_kernel<<<dim3((N + 31) / 32, H), 256, smem, stream>>>((const bf16*)x, xs_t, xs_h, (const bf16*)w,
                                                                          (bf16*)out, os_t, os_h, M, N, K);
    return q3_launch_status();
  }
  if (dtype == Q3_DTYPE_F32) return launch_head_gemm<float>(x, xs_t, xs_h, w, out, os_t, os_h, M, H, N, K, stream);
  if (dtype == Q3_DTYPE_BF16) return launch_head_gemm<bf16>(x, xs_t, xs_h, w, out, os_t, os_h, M, H, N, K, stream);
  return Q3_ERR_ARGUMENT;
}
