// Linear attention with a decayed matrix state per (sequence, head), kept in fp32 in a state slot:
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T        o_t = S_t^T q_t        S: [D, Dv]
//
// a_t is a decay per key channel.  It comes either from logits, a_t[i] = sigmoid(z_t[i] + b[i])^(1 / tau)
// (gated linear attention), or is one constant per head (retention).  q and k may be rotated first
// (pairs (i, i + pairs) of a head turn by position * inv_freq[i]) and are multiplied by q_scale and
// k_scale; decays, angles, the state and the products with it are fp32, q, k, v and z arrive in the
// activation type.
//
// decayed_state_scan: one block per (32 value columns, head, sequence).  Lane = value column, warp =
// group of R key rows, so a thread keeps R elements of the state in registers from the sequence's
// first token of the step to its last.  Tokens are staged CT at a time in shared memory (q, k and
// decay rows as fp32, already rotated and scaled), every thread runs the CT updates on its rows, the
// warps' partial outputs are added in warp order.  A token's arithmetic does not depend on where
// the step's portion starts or ends, so the result has the same bits however a prompt is cut.
//
// head_norm_gate: y[t, h, :] = o / sqrt(mean(o^2) + eps) * w * silu(g[t, h, :]) * out_scale, one warp
// per (token, head); w may be absent.
#include "common.cuh"

#define SCAN_CT 8   // tokens staged at a time
#define SCAN_R 8    // key rows per thread

template <typename T>
__global__ void __launch_bounds__(1024)
decayed_state_scan_kernel(const T* __restrict__ q, long q_stride, const T* __restrict__ k, long k_stride,
                          const T* __restrict__ v, long v_stride, const T* __restrict__ z, long z_stride,
                          const float* __restrict__ z_bias, float inv_tau, const float* __restrict__ head_decay,
                          const float* __restrict__ inv_freq, int rot_pairs, const int* __restrict__ positions,
                          float q_scale, float k_scale, float* __restrict__ state,
                          const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                          float* __restrict__ out, int H, int D, int Dv) {
  extern __shared__ __align__(16) float scan_smem[];
  const int nwarp = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int Dp = nwarp * SCAN_R;                 // D rounded up to the rows the block holds
  float* qs = scan_smem;                          // [CT][Dp]
  float* ks = qs + SCAN_CT * Dp;                  // [CT][Dp]
  float* as = ks + SCAN_CT * Dp;                  // [CT][Dp]
  float* vs = as + SCAN_CT * Dp;                  // [CT][32]
  float* part = vs + SCAN_CT * 32;                // [nwarp][CT][32]
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.y, b = blockIdx.z;
  const int j = blockIdx.x * 32 + lane;
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  const long slot = state_slots[b];
  float* Sg = state + ((slot * H + h) * (long)D) * Dv;
  float S[SCAN_R];
#pragma unroll
  for (int r = 0; r < SCAN_R; ++r) {
    const int i = warp * SCAN_R + r;
    S[r] = (i < D && j < Dv) ? Sg[(long)i * Dv + j] : 0.f;
  }
  const float decay_h = head_decay ? head_decay[h] : 1.f;
  for (int c0 = t0; c0 < t1; c0 += SCAN_CT) {
    const int n = min(SCAN_CT, t1 - c0);
    // stage the chunk: rows beyond D are zero (their state stays zero and adds nothing)
    for (int x = threadIdx.x; x < n * Dp; x += blockDim.x) {
      const int c = x / Dp, i = x - c * Dp;
      const long t = c0 + c;
      float qv = 0.f, kv = 0.f, av = 0.f;
      if (i < D) {
        qv = to_f32(q[t * q_stride + h * D + i]);
        kv = to_f32(k[t * k_stride + h * D + i]);
        if (i < 2 * rot_pairs) {
          const int pair = i < rot_pairs ? i : i - rot_pairs;
          const int other = i < rot_pairs ? i + rot_pairs : i - rot_pairs;
          float sn, cs;
          sincosf((float)positions[t] * inv_freq[pair], &sn, &cs);
          const float qo = to_f32(q[t * q_stride + h * D + other]);
          const float ko = to_f32(k[t * k_stride + h * D + other]);
          // first of a pair: u cos - v sin; second: v cos + u sin
          qv = i < rot_pairs ? qv * cs - qo * sn : qv * cs + qo * sn;
          kv = i < rot_pairs ? kv * cs - ko * sn : kv * cs + ko * sn;
        }
        qv *= q_scale;
        kv *= k_scale;
        if (z) {
          const float zz = to_f32(z[t * z_stride + h * D + i]) + (z_bias ? z_bias[h * D + i] : 0.f);
          const float log_sig = fminf(zz, 0.f) - log1pf(expf(-fabsf(zz)));
          av = expf(log_sig * inv_tau);
        } else {
          av = decay_h;
        }
      }
      qs[x] = qv;
      ks[x] = kv;
      as[x] = av;
    }
    for (int x = threadIdx.x; x < n * 32; x += blockDim.x) {
      const int c = x >> 5, jj = blockIdx.x * 32 + (x & 31);
      vs[x] = jj < Dv ? to_f32(v[(long)(c0 + c) * v_stride + h * Dv + jj]) : 0.f;
    }
    __syncthreads();
    const int i0 = warp * SCAN_R;
    for (int c = 0; c < n; ++c) {
      const float vj = vs[c * 32 + lane];
      const float4* a4 = reinterpret_cast<const float4*>(as + c * Dp + i0);
      const float4* k4 = reinterpret_cast<const float4*>(ks + c * Dp + i0);
      const float4* q4 = reinterpret_cast<const float4*>(qs + c * Dp + i0);
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int g = 0; g < SCAN_R / 4; ++g) {
        const float4 a = a4[g], kk = k4[g], qq = q4[g];
        S[4 * g + 0] = fmaf(a.x, S[4 * g + 0], kk.x * vj);
        S[4 * g + 1] = fmaf(a.y, S[4 * g + 1], kk.y * vj);
        S[4 * g + 2] = fmaf(a.z, S[4 * g + 2], kk.z * vj);
        S[4 * g + 3] = fmaf(a.w, S[4 * g + 3], kk.w * vj);
        acc0 = fmaf(S[4 * g + 0], qq.x, acc0);
        acc1 = fmaf(S[4 * g + 1], qq.y, acc1);
        acc0 = fmaf(S[4 * g + 2], qq.z, acc0);
        acc1 = fmaf(S[4 * g + 3], qq.w, acc1);
      }
      part[(warp * SCAN_CT + c) * 32 + lane] = acc0 + acc1;
    }
    __syncthreads();
    for (int x = threadIdx.x; x < n * 32; x += blockDim.x) {
      const int c = x >> 5, jj = blockIdx.x * 32 + (x & 31);
      float sum = 0.f;
      for (int w = 0; w < nwarp; ++w) sum += part[(w * SCAN_CT + c) * 32 + (x & 31)];
      if (jj < Dv) out[((long)(c0 + c) * H + h) * Dv + jj] = sum;
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < SCAN_R; ++r) {
    const int i = warp * SCAN_R + r;
    if (i < D && j < Dv) Sg[(long)i * Dv + j] = S[r];
  }
}

// q, k: head h of token t at [t * stride + h * D]; v at [t * v_stride + h * Dv]; z (decay logits, or
// null) like q, z_bias fp32 [H * D] or null; head_decay fp32 [H] (used when z is null); inv_freq fp32
// [rot_pairs] with positions, or rot_pairs = 0; state fp32 [slots, H, D, Dv]; out fp32 [T, H, Dv].
Q3_EXPORT int q3_decayed_state_scan(int dtype, const void* q, long q_stride, const void* k, long k_stride,
                                    const void* v, long v_stride, const void* z, long z_stride, const float* z_bias,
                                    float inv_tau, const float* head_decay, const float* inv_freq, int rot_pairs,
                                    const int* positions, float q_scale, float k_scale, float* state,
                                    const int* cu_seqlens, const int* state_slots, float* out, int num_seqs, int H,
                                    int D, int Dv, cudaStream_t stream) {
  if (!q || !k || !v || !state || !cu_seqlens || !state_slots || !out) return Q3_ERR_ARGUMENT;
  if (!z && !head_decay) return Q3_ERR_ARGUMENT;
  if (rot_pairs < 0 || 2 * rot_pairs > D || (rot_pairs && (!inv_freq || !positions))) return Q3_ERR_ARGUMENT;
  if (H < 1 || D < 1 || Dv < 1 || H > 65535 || num_seqs > 65535) return Q3_ERR_ARGUMENT;
  if (D > 32 * SCAN_R) return Q3_ERR_UNSUPPORTED;
  if (num_seqs == 0) return Q3_OK;
  const int nwarp = (D + SCAN_R - 1) / SCAN_R;
  const int Dp = nwarp * SCAN_R;
  const size_t smem = (size_t)(3 * SCAN_CT * Dp + SCAN_CT * 32 + nwarp * SCAN_CT * 32) * sizeof(float);
  const dim3 grid((Dv + 31) / 32, H, num_seqs);
  cudaError_t e;
  if (dtype == Q3_DTYPE_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(decayed_state_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    e = launch_pdl(decayed_state_scan_kernel<float>, grid, dim3(32 * nwarp), smem, stream, (const float*)q, q_stride,
                   (const float*)k, k_stride, (const float*)v, v_stride, (const float*)z, z_stride, z_bias, inv_tau,
                   head_decay, inv_freq, rot_pairs, positions, q_scale, k_scale, state, cu_seqlens, state_slots, out, H,
                   D, Dv);
  } else if (dtype == Q3_DTYPE_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(decayed_state_scan_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    e = launch_pdl(decayed_state_scan_kernel<bf16>, grid, dim3(32 * nwarp), smem, stream, (const bf16*)q, q_stride,
                   (const bf16*)k, k_stride, (const bf16*)v, v_stride, (const bf16*)z, z_stride, z_bias, inv_tau,
                   head_decay, inv_freq, rot_pairs, positions, q_scale, k_scale, state, cu_seqlens, state_slots, out, H,
                   D, Dv);
  } else {
    return Q3_ERR_ARGUMENT;
  }
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}

template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps,
                                      const T* __restrict__ g, long g_stride, T* __restrict__ y, long y_stride,
                                      float out_scale, long items, int H, int Dv) {
  pdl_wait();
  pdl_launch_dependents();
  const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= items) return;
  const long t = item / H;
  const int h = (int)(item - t * H);
  const float* orow = o + item * Dv;
  float ss = 0.f;
  for (int d = lane; d < Dv; d += 32) ss += orow[d] * orow[d];
  const float rstd = rsqrtf(warp_sum(ss) / (float)Dv + eps);
  const T* grow = g + t * g_stride + (long)h * Dv;
  T* yrow = y + t * y_stride + (long)h * Dv;
  for (int d = lane; d < Dv; d += 32) {
    float val = orow[d] * rstd;
    if (w) val *= w[d];
    const float gate = to_f32(grow[d]);
    yrow[d] = from_f32<T>(val * (gate / (1.f + expf(-gate))) * out_scale);
  }
}

// o: fp32 [T, H, Dv]; w: fp32 [Dv] shared by the heads, or null; g, y: head h of token t at
// [t * stride + h * Dv].
Q3_EXPORT int q3_head_norm_gate(int dtype, const float* o, const float* w, float eps, const void* g, long g_stride,
                                void* y, long y_stride, float out_scale, int num_tokens, int H, int Dv,
                                cudaStream_t stream) {
  if (!o || !g || !y || H < 1 || Dv < 1) return Q3_ERR_ARGUMENT;
  const long items = (long)num_tokens * H;
  if (items == 0) return Q3_OK;
  const unsigned blocks = (unsigned)((items + 7) / 8);
  cudaError_t e;
  if (dtype == Q3_DTYPE_F32)
    e = launch_pdl(head_norm_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, o, w, eps, (const float*)g,
                   g_stride, (float*)y, y_stride, out_scale, items, H, Dv);
  else if (dtype == Q3_DTYPE_BF16)
    e = launch_pdl(head_norm_gate_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, o, w, eps, (const bf16*)g, g_stride,
                   (bf16*)y, y_stride, out_scale, items, H, Dv);
  else
    return Q3_ERR_ARGUMENT;
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}
