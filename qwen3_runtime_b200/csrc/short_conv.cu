// A short causal convolution over time on every channel of a fused q/k/v projection, followed by
// what the attention needs of its result: rotation of q and k, and the write of k and v into their
// cache pages.
//
//   y_t[c] = sum_j w[c, j] * u_(t - taps + 1 + j)[c]          (zeros before the sequence's start)
//
// u is the projection's output.  The last taps - 1 rows of u of every sequence live in a state slot
// (fp32 [taps - 1, C], row m holds position start - (taps - 1) + m), so that a step continues where
// the last one stopped; conv_state_update writes them after conv_rope_store has read the old ones.
// The convolution accumulates in fp32 in tap order; its result is rotated in fp32 and rounded once.
//
// conv_rope_store: one thread per (token, work item); a work item is a rotation pair (i, i + pairs) of
// four q or k heads in a row, an element of such heads that does not turn, or an element of four v
// heads, so that no thread waits for another and every thread's loads are in flight at once.
//   q heads: pairs (i, i + pairs) of a head turn by position * inv_freq[i], written to q_out
//   k heads: the same, written to the token's row of k_pages
//   v heads: multiplied by value_scale, written to the token's row of v_pages
// Keys have D elements a head, values Dv.
#include "common.cuh"

#define CONV_MAX_TAPS 16

// One channel's convolution at token `t` of the step, which is `n` rows into its sequence's portion.
// The step's own rows are read whether or not they belong to the sequence (never before row 0 of the
// step), so that these loads wait for nothing; the few rows that come from the state replace them.
// TAPS > 0: the tap count at compile time, the loop unrolled, so that all loads are in flight at once;
// TAPS < 0: any count (`taps`).
template <typename T, int TAPS>
__device__ __forceinline__ float conv_channel(const T* __restrict__ xrow, long x_stride, const float* __restrict__ w,
                                              int taps, const float* __restrict__ srow, int C, int t, int n, int c) {
  if (TAPS == 0) return to_f32(xrow[c]);
  if (TAPS > 0) {
    float u[TAPS > 0 ? TAPS : 1], wj[TAPS > 0 ? TAPS : 1];
#pragma unroll
    for (int j = 0; j < TAPS; ++j) {
      const int back = TAPS - 1 - j;  // how many tokens before this one
      u[j] = to_f32(xrow[-(long)min(back, t) * x_stride + c]);
      wj[j] = w[(long)j * C + c];
    }
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < TAPS; ++j) {
      const int back = TAPS - 1 - j;
      if (n - back < 0) u[j] = srow[(long)(TAPS - 1 + n - back) * C + c];
      acc = fmaf(wj[j], u[j], acc);
    }
    return acc;
  }
  float acc = 0.f;
  for (int j = 0; j < taps; ++j) {
    const int back = taps - 1 - j;
    float u = to_f32(xrow[-(long)min(back, t) * x_stride + c]);
    if (n - back < 0) u = srow[(long)(taps - 1 + n - back) * C + c];
    acc = fmaf(w[(long)j * C + c], u, acc);
  }
  return acc;
}

// A thread takes one work item of CONV_HG heads in a row: with four (steps of many tokens) the loads of
// all of them are in flight together, their angle is worked out once, and the step's tokens pass in a
// quarter of the blocks; with one (a few tokens) a thread's chain is shortest.
template <typename T, int TAPS, int CONV_HG>
__global__ void __launch_bounds__(256)
conv_rope_store_kernel(const T* __restrict__ x, long x_stride, const float* __restrict__ w, int taps,
                       const float* __restrict__ conv_state, const int* __restrict__ positions,
                       const int* __restrict__ token_seq, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ state_slots, const float* __restrict__ inv_freq, int rot_pairs,
                       T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages,
                       const int* __restrict__ block_table, int max_pages, int ps, int nq, int nkv, int D, int Dv,
                       float value_scale, int write_kv) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int item = blockIdx.y * blockDim.x + threadIdx.x;
  const int per_head = D - rot_pairs;  // work items of a q or k head: its pairs, then what does not turn
  const int qk_groups = (nq + nkv + CONV_HG - 1) / CONV_HG, v_groups = (nkv + CONV_HG - 1) / CONV_HG;
  const int qk_items = qk_groups * per_head;
  if (item >= qk_items + v_groups * Dv) return;
  const int b = token_seq[t];
  const int p = positions[t];
  const int Cq = nq * D, Ck = nkv * D, C = Cq + Ck + nkv * Dv;
  const int n = t - cu_seqlens[b];  // the token's place in its sequence's portion
  const T* xrow = x + (long)t * x_stride;
  const float* srow = taps > 1 ? conv_state + (long)state_slots[b] * (taps - 1) * C : nullptr;
  const int page = write_kv ? block_table[(long)b * max_pages + p / ps] : 0;
  const long page_row = (long)page * nkv * ps + p % ps;  // head 0's row of the token in its page
  if (item >= qk_items) {  // element e of CONV_HG v heads
    if (!write_kv) return;
    const int vi = item - qk_items, group = vi / Dv, e = vi - group * Dv;
    float y[CONV_HG];
#pragma unroll
    for (int hh = 0; hh < CONV_HG; ++hh) {
      const int head = group * CONV_HG + hh;
      y[hh] = head < nkv ? conv_channel<T, TAPS>(xrow, x_stride, w, taps, srow, C, t, n, Cq + Ck + head * Dv + e) : 0.f;
    }
#pragma unroll
    for (int hh = 0; hh < CONV_HG; ++hh) {
      const int head = group * CONV_HG + hh;
      if (head < nkv) v_pages[(page_row + (long)head * ps) * Dv + e] = from_f32<T>(y[hh] * value_scale);
    }
    return;
  }
  const int group = item / per_head, r = item - group * per_head;  // q heads, then k heads
  const bool turns = r < rot_pairs;
  const int e = turns ? r : r + rot_pairs;  // the element (the first of its pair, if it turns)
  float u[CONV_HG], v[CONV_HG];
#pragma unroll
  for (int hh = 0; hh < CONV_HG; ++hh) {
    const int head = group * CONV_HG + hh;
    const bool live = head < nq + nkv && (head < nq || write_kv);
    u[hh] = live ? conv_channel<T, TAPS>(xrow, x_stride, w, taps, srow, C, t, n, head * D + e) : 0.f;
    v[hh] = live && turns ? conv_channel<T, TAPS>(xrow, x_stride, w, taps, srow, C, t, n, head * D + e + rot_pairs) : 0.f;
  }
  float sn = 0.f, cs = 1.f;
  if (turns) sincosf((float)p * inv_freq[r], &sn, &cs);
#pragma unroll
  for (int hh = 0; hh < CONV_HG; ++hh) {
    const int head = group * CONV_HG + hh;
    if (head >= nq + nkv || (head >= nq && !write_kv)) continue;
    T* dst = head < nq ? q_out + (long)t * Cq + (long)head * D : k_pages + (page_row + (long)(head - nq) * ps) * D;
    if (turns) {
      dst[e] = from_f32<T>(u[hh] * cs - v[hh] * sn);
      dst[e + rot_pairs] = from_f32<T>(v[hh] * cs + u[hh] * sn);
    } else {
      dst[e] = from_f32<T>(u[hh]);
    }
  }
}

// x: [T, C] rows x_stride apart, C = nq * D + nkv * D + nkv * Dv (q heads, k heads, v heads); w: fp32
// [taps, C], tap-major so that neighbouring channels' weights are neighbours (taps = 0: no convolution, conv_state unused); conv_state: fp32 [slots, taps - 1, C];
// inv_freq: fp32 [rot_pairs] or rot_pairs = 0; q_out: dense [T, nq * D]; k_pages [pages, nkv, ps, D],
// v_pages [pages, nkv, ps, Dv].
Q3_EXPORT int q3_conv_rope_store(int dtype, const void* x, long x_stride, const float* w, int taps,
                                 const float* conv_state, const int* positions, const int* token_seq,
                                 const int* cu_seqlens, const int* state_slots, const float* inv_freq, int rot_pairs,
                                 void* q_out, void* k_pages, void* v_pages, const int* block_table, int max_pages,
                                 int ps, int num_tokens, int nq, int nkv, int D, int Dv, float value_scale,
                                 int write_kv, cudaStream_t stream) {
  if (!x || !positions || !token_seq || !cu_seqlens || !q_out) return Q3_ERR_ARGUMENT;
  if (taps < 0 || taps > CONV_MAX_TAPS) return Q3_ERR_UNSUPPORTED;
  if (taps > 0 && (!w || !state_slots || (taps > 1 && !conv_state))) return Q3_ERR_ARGUMENT;
  if (write_kv && (!k_pages || !v_pages || !block_table || ps < 1)) return Q3_ERR_ARGUMENT;
  if (nq < 1 || nkv < 1 || D < 1 || Dv < 1 || rot_pairs < 0 || 2 * rot_pairs > D || (rot_pairs && !inv_freq))
    return Q3_ERR_ARGUMENT;
  if (num_tokens == 0) return Q3_OK;
  const int hg = num_tokens > 64 ? 4 : 1;  // heads per thread
  const int items = ((nq + nkv + hg - 1) / hg) * (D - rot_pairs) + ((nkv + hg - 1) / hg) * Dv;
  if ((items + 255) / 256 > 65535) return Q3_ERR_UNSUPPORTED;
  const dim3 grid(num_tokens, (items + 255) / 256);
  cudaError_t e = cudaErrorInvalidValue;
#define Q3_CONV_HG(T, TAPS, HG)                                                                                      \
  e = launch_pdl(conv_rope_store_kernel<T, TAPS, HG>, grid, dim3(256), 0, stream, (const T*)x, x_stride, w, taps,    \
                 conv_state, positions, token_seq, cu_seqlens, state_slots, inv_freq, rot_pairs, (T*)q_out,          \
                 (T*)k_pages, (T*)v_pages, block_table, max_pages, ps, nq, nkv, D, Dv, value_scale, write_kv)
#define Q3_CONV(T, TAPS)                                                                                             \
  if (hg == 4) Q3_CONV_HG(T, TAPS, 4); else Q3_CONV_HG(T, TAPS, 1)
#define Q3_CONV_TAPS(T)                                                                                              \
  switch (taps) {                                                                                                    \
    case 0: Q3_CONV(T, 0); break;                                                                                    \
    case 1: Q3_CONV(T, 1); break;                                                                                    \
    case 2: Q3_CONV(T, 2); break;                                                                                    \
    case 3: Q3_CONV(T, 3); break;                                                                                    \
    case 4: Q3_CONV(T, 4); break;                                                                                    \
    default: Q3_CONV(T, -1); break;                                                                                  \
  }
  if (dtype == Q3_DTYPE_F32) {
    Q3_CONV_TAPS(float)
  } else if (dtype == Q3_DTYPE_BF16) {
    Q3_CONV_TAPS(bf16)
  } else {
    return Q3_ERR_ARGUMENT;
  }
#undef Q3_CONV_TAPS
#undef Q3_CONV
#undef Q3_CONV_HG
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}

// The last taps - 1 rows of u of every sequence after this step: rows of the step where it brought
// enough, else older rows of the state moved up.  One thread per (sequence, channel) reads all it
// needs before it writes.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ x, long x_stride, float* __restrict__ conv_state,
                                         const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                                         int taps, int C, int num_seqs) {
  pdl_wait();
  pdl_launch_dependents();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)num_seqs * C) return;
  const int b = (int)(idx / C), c = (int)(idx - (long)b * C);
  const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
  float* srow = conv_state + (long)state_slots[b] * (taps - 1) * C;
  float keep[CONV_MAX_TAPS];
#pragma unroll
  for (int m = 0; m < CONV_MAX_TAPS - 1; ++m) {
    if (m >= taps - 1) break;
    const int li = n - (taps - 1) + m;  // the row's place in this step's portion
    keep[m] = li >= 0 ? to_f32(x[(long)(t0 + li) * x_stride + c]) : srow[(long)(m + n) * C + c];
  }
#pragma unroll
  for (int m = 0; m < CONV_MAX_TAPS - 1; ++m) {
    if (m >= taps - 1) break;
    srow[(long)m * C + c] = keep[m];
  }
}

Q3_EXPORT int q3_conv_state_update(int dtype, const void* x, long x_stride, float* conv_state, const int* cu_seqlens,
                                   const int* state_slots, int taps, int C, int num_seqs, cudaStream_t stream) {
  if (!x || !conv_state || !cu_seqlens || !state_slots || C < 1) return Q3_ERR_ARGUMENT;
  if (taps < 2) return Q3_OK;  // nothing is carried
  if (taps > CONV_MAX_TAPS) return Q3_ERR_UNSUPPORTED;
  const long total = (long)num_seqs * C;
  if (total == 0) return Q3_OK;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaError_t e;
  if (dtype == Q3_DTYPE_F32)
    e = launch_pdl(conv_state_update_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)x, x_stride,
                   conv_state, cu_seqlens, state_slots, taps, C, num_seqs);
  else if (dtype == Q3_DTYPE_BF16)
    e = launch_pdl(conv_state_update_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)x, x_stride,
                   conv_state, cu_seqlens, state_slots, taps, C, num_seqs);
  else
    return Q3_ERR_ARGUMENT;
  return e == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}
