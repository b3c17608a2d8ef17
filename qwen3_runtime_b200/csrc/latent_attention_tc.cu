// Attention over latent rows on the tensor cores (bfloat16, mma.sync m16n8k16), for prompt portions
// and single decoded tokens alike.  The cache holds one row [latent | rotated key part] of dk
// elements per token for all heads, the value of a row is its first dv elements, and queries
// arrive already in the rows' space -- see latent_attention.cu, whose kernel is the fp32 path and
// takes the sizes this one refuses.
//
// A block owns 32 (token, head) rows of one sequence: `hgp` heads (the head count rounded up to a
// power of two, at most 32) of 32 / hgp consecutive tokens, so that all its rows read nearly the
// same keys.  Keys come in tiles of 64 rows through cp.async into shared memory, once for all the
// block's rows, the next tile on its way while one is worked on (two buffers, where they fit).  Per tile:
//   1. S = Q K^T: each of the eight warps scores 16 of the tile's keys for 16 of the rows (Q and K
//      fragments by ldmatrix, the reduction over dk in steps of 16), scaled fp32 scores go to shared
//      memory;
//   2. softmax: eight threads per row mask (causal, window), take the running maximum and sum in
//      fp32 with exact expf, and leave P as bfloat16 and the rescale factor in shared memory;
//   3. O = O * rescale + P V: a warp owns 16 rows and a quarter of the value columns, with V read
//      from the same key tile through ldmatrix.trans.
// A sink starts a row's running maximum at sink_h with a denominator of 1 and no value.
//
// In a step where every sequence brings one token there are few rows and many keys: the keys of a
// sequence are then cut into `splits` slices of whole tiles, a block per slice leaves its
// unnormalised O with its maximum and denominator in a scratch, and a second kernel merges the
// slices (the sink belongs to slice 0).
#include "mma_tiles.cuh"

constexpr int LTC_BM = 32, LTC_BN = 64, LTC_THREADS = 256;
constexpr int LTC_SS = LTC_BN + 4;  // fp32 score row stride
constexpr int LTC_PS = LTC_BN + 8;  // bf16 probability row stride (ldmatrix rows 16 bytes apart in banks)

template <int NT>  // value tiles of 8 columns per warp: dv <= 32 * NT
__global__ void __launch_bounds__(LTC_THREADS)
latent_attention_tc_kernel(const bf16* __restrict__ q, long qs_t, long qs_h, const bf16* __restrict__ pages, int dk,
                           int dv, const int* __restrict__ block_table, int max_pages,
                           const int* __restrict__ cu_seqlens, const int* __restrict__ kv_lens,
                           const float* __restrict__ sink, bf16* __restrict__ out, long os_t, long os_h, int H,
                           int hgp, int ps, float scale, int window, int splits, float* __restrict__ part,
                           int stages) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int kstride = dk + 8;  // elements; rows stay 16-byte aligned and ldmatrix is conflict-free
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                 // [32][kstride]
  bf16* Kbuf = Qs + LTC_BM * kstride;                           // [stages][64][kstride]
  float* Ss = reinterpret_cast<float*>(Kbuf + stages * LTC_BN * kstride);  // [32][LTC_SS]
  bf16* Ps = reinterpret_cast<bf16*>(Ss + LTC_BM * LTC_SS);     // [32][LTC_PS]
  float* row_m = reinterpret_cast<float*>(Ps + LTC_BM * LTC_PS);
  float* row_l = row_m + LTC_BM;
  float* row_c = row_l + LTC_BM;
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z;
  const int tq = LTC_BM / hgp;  // tokens per block
  const int seq_start = cu_seqlens[b], seq_len = cu_seqlens[b + 1] - seq_start;
  const int split = splits > 1 ? blockIdx.x : 0;  // with slices a sequence brings one token: one row tile
  const int t_local0 = splits > 1 ? 0 : blockIdx.x * tq;
  if (t_local0 >= seq_len) return;
  const int ntok = min(tq, seq_len - t_local0);
  const int head0 = blockIdx.y * hgp;
  const int pos0 = kv_lens[b] - seq_len + t_local0;  // position of the block's first token
  const int j_hi = pos0 + ntok - 1;
  const int j_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int* bt = block_table + (long)b * max_pages;
  const int chunks = dk >> 3;

  // queries of the block's rows; rows without a token or a head are zero
  for (int c = tid; c < LTC_BM * chunks; c += LTC_THREADS) {
    const int r = c / chunks, ch = c - r * chunks;
    const int tl = r / hgp, head = head0 + (r - tl * hgp);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tl < ntok && head < H)
      v = *reinterpret_cast<const uint4*>(q + (long)(seq_start + t_local0 + tl) * qs_t + (long)head * qs_h + ch * 8);
    *reinterpret_cast<uint4*>(Qs + r * kstride + ch * 8) = v;
  }
  if (tid < LTC_BM) {
    const int tl = tid / hgp, head = head0 + (tid - tl * hgp);
    const bool live = tl < ntok && head < H;
    row_m[tid] = (live && sink && split == 0) ? sink[head] : -INFINITY;
    row_l[tid] = (live && sink && split == 0) ? 1.f : 0.f;
  }
  const int mt = warp >> 2;  // this warp's 16 rows
  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
  const int ncol0 = (warp & 3) * NT * 8;  // this warp's first value column
  int j_begin = j_lo, j_end = j_hi;       // this block's keys
  if (splits > 1) {
    const int tiles = (j_hi - j_lo) / LTC_BN + 1, per = (tiles + splits - 1) / splits;
    j_begin = j_lo + split * per * LTC_BN;
    j_end = min(j_hi, j_begin + per * LTC_BN - 1);
  }

  // one tile of keys into a buffer: rows beyond the block's last key, and rows of released pages, as zeros
  auto load_tile = [&](int j0, bf16* dst) {
    // four threads per key row: one page lookup a thread, then 16-byte chunks four apart
    const int jj = tid >> 2, j = j0 + jj;
    const bf16* src = pages;
    int bytes = 0;
    if (j <= j_hi) {
      const int page = bt[j / ps];
      if (page >= 0) {
        src = pages + ((long)page * ps + (j % ps)) * dk;
        bytes = 16;
      }
    }
    const uint32_t drow = smem_u32(dst + jj * kstride);
    for (int ch = tid & 3; ch < chunks; ch += 4)
      cp_async16(drow + ch * 16, bytes ? src + ch * 8 : src, bytes);  // 0 bytes: the chunk is zero-filled
    cp_async_commit();
  };
  // With two buffers the next tile is on its way while this one is worked on.
  if (stages > 1 && j_begin <= j_end) load_tile(j_begin, Kbuf);
  int it = 0;
  for (int j0 = j_begin; j0 <= j_end; j0 += LTC_BN, ++it) {
    bf16* Ks = Kbuf + (stages > 1 ? (it & 1) : 0) * LTC_BN * kstride;
    if (stages > 1) {
      cp_async_wait<0>();
      __syncthreads();  // this tile has landed; the tile before it has been used up (and Qs / row state are written)
      if (j0 + LTC_BN <= j_end) load_tile(j0 + LTC_BN, Kbuf + ((it + 1) & 1) * LTC_BN * kstride);
    } else {
      __syncthreads();  // the tile before this one has been used up (and Qs / row state are written)
      load_tile(j0, Ks);
      cp_async_wait<0>();
      __syncthreads();
    }

    // 1. scores of 16 keys for this warp's 16 rows
    {
      float sc[2][4], sd[2][4];  // even and odd steps of the reduction: two chains of dependent MMAs
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[nt][e] = sd[nt][e] = 0.f;
      const int key0 = (warp & 3) * 16;
      const int a_row = mt * 16 + (lane & 15), a_col = (lane >> 4) * 8;
      const int b_row = key0 + ((lane >> 4) * 8) + (lane & 7), b_col = ((lane >> 3) & 1) * 8;
      const uint32_t a_addr = smem_u32(Qs + a_row * kstride + a_col), b_addr = smem_u32(Ks + b_row * kstride + b_col);
      int k0 = 0;
#pragma unroll 2
      for (; k0 + 32 <= dk; k0 += 32) {
        uint32_t a0[4], b0[4], a1[4], b1[4];
        ldmatrix_x4(a0, a_addr + k0 * 2);
        ldmatrix_x4(b0, b_addr + k0 * 2);
        ldmatrix_x4(a1, a_addr + k0 * 2 + 32);
        ldmatrix_x4(b1, b_addr + k0 * 2 + 32);
        mma_bf16(sc[0], a0, b0[0], b0[1]);
        mma_bf16(sc[1], a0, b0[2], b0[3]);
        mma_bf16(sd[0], a1, b1[0], b1[1]);
        mma_bf16(sd[1], a1, b1[2], b1[3]);
      }
      if (k0 < dk) {  // dk is a multiple of 16: one step is left
        uint32_t a0[4], b0[4];
        ldmatrix_x4(a0, a_addr + k0 * 2);
        ldmatrix_x4(b0, b_addr + k0 * 2);
        mma_bf16(sc[0], a0, b0[0], b0[1]);
        mma_bf16(sc[1], a0, b0[2], b0[3]);
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[nt][e] += sd[nt][e];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int r = mt * 16 + (lane >> 2), cidx = key0 + nt * 8 + 2 * (lane & 3);
        Ss[r * LTC_SS + cidx] = sc[nt][0] * scale;
        Ss[r * LTC_SS + cidx + 1] = sc[nt][1] * scale;
        Ss[(r + 8) * LTC_SS + cidx] = sc[nt][2] * scale;
        Ss[(r + 8) * LTC_SS + cidx + 1] = sc[nt][3] * scale;
      }
    }
    __syncthreads();

    // 2. softmax of the tile: eight threads per row, 8 keys each
    {
      const int r = tid >> 3, part = tid & 7;
      const int tl = r / hgp, head = head0 + (r - tl * hgp);
      const bool live = tl < ntok && head < H;
      const int pos = pos0 + tl;
      const int lo = window > 0 ? max(0, pos - window + 1) : 0;
      float sv[8];
      float mx = -INFINITY;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int j = j0 + part * 8 + e;
        const bool seen = live && j >= lo && j <= pos;
        sv[e] = seen ? Ss[r * LTC_SS + part * 8 + e] : -INFINITY;
        mx = fmaxf(mx, sv[e]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      const float m_old = row_m[r];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      __nv_bfloat162* prow = reinterpret_cast<__nv_bfloat162*>(Ps + r * LTC_PS + part * 8);
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        const float p0 = sv[e] == -INFINITY ? 0.f : expf(sv[e] - m_new);
        const float p1 = sv[e + 1] == -INFINITY ? 0.f : expf(sv[e + 1] - m_new);
        sum += p0 + p1;
        prow[e >> 1] = __floats2bfloat162_rn(p0, p1);
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      __syncwarp();  // every thread of the row has read row_m before it is replaced
      if (part == 0) {
        const float corr = m_new == -INFINITY ? 1.f : expf(m_old - m_new);
        row_c[r] = corr;
        row_l[r] = row_l[r] * corr + sum;
        row_m[r] = m_new;
      }
    }
    __syncthreads();

    // 3. O = O * rescale + P V on this warp's rows and value columns
    {
      const float c_lo = row_c[mt * 16 + (lane >> 2)], c_hi = row_c[mt * 16 + 8 + (lane >> 2)];
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        o[i][0] *= c_lo;
        o[i][1] *= c_lo;
        o[i][2] *= c_hi;
        o[i][3] *= c_hi;
      }
      const int a_row = mt * 16 + (lane & 15), a_col = (lane >> 4) * 8;
      const int v_row = ((lane >> 3) & 1) * 8 + (lane & 7), v_col = (lane >> 4) * 8;
#pragma unroll
      for (int kk0 = 0; kk0 < LTC_BN; kk0 += 16) {
        uint32_t a[4];
        ldmatrix_x4(a, smem_u32(Ps + a_row * LTC_PS + kk0 + a_col));
#pragma unroll
        for (int i = 0; i < NT; i += 2) {
          const int n = ncol0 + i * 8;
          if (n >= dv) continue;  // dv is a multiple of 16: a pair of tiles is inside or outside
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, smem_u32(Ks + (kk0 + v_row) * kstride + n + v_col));
          mma_bf16(o[i], a, vb[0], vb[1]);
          mma_bf16(o[i + 1], a, vb[2], vb[3]);
        }
      }
    }
  }
  __syncthreads();  // row_m / row_l of the last tile
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = mt * 16 + half * 8 + (lane >> 2);
    const int tl = r / hgp, head = head0 + (r - tl * hgp);
    if (tl >= ntok || head >= H) continue;
    if (splits > 1) {  // this slice's share: unnormalised values, then (once per row) maximum and denominator
      float* dst = part + (((long)b * H + head) * splits + split) * (dv + 2);
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const int n = ncol0 + i * 8 + 2 * (lane & 3);
        if (n < dv) {
          dst[n] = o[i][2 * half];
          dst[n + 1] = o[i][2 * half + 1];
        }
      }
      if ((warp & 3) == 0 && (lane & 3) == 0) {
        dst[dv] = row_m[r];
        dst[dv + 1] = row_l[r];
      }
      continue;
    }
    const float inv = 1.f / row_l[r];
    bf16* orow = out + (long)(seq_start + t_local0 + tl) * os_t + (long)head * os_h;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int n = ncol0 + i * 8 + 2 * (lane & 3);
      if (n < dv)
        *reinterpret_cast<__nv_bfloat162*>(orow + n) = __floats2bfloat162_rn(o[i][2 * half] * inv, o[i][2 * half + 1] * inv);
    }
  }
}

// The slices of one (sequence, head): out = sum_s o_s e^(m_s - M) / sum_s l_s e^(m_s - M), M = max_s m_s.
__global__ void latent_attention_merge_kernel(const float* __restrict__ part, const int* __restrict__ cu_seqlens,
                                              bf16* __restrict__ out, long os_t, long os_h, int H, int dv,
                                              int splits) {
  __shared__ float wgt[64];
  __shared__ float inv_l;
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x / H, head = blockIdx.x % H;
  const float* src = part + (long)blockIdx.x * splits * (dv + 2);
  if (threadIdx.x == 0) {
    float M = -INFINITY;
    for (int sp = 0; sp < splits; ++sp) M = fmaxf(M, src[(long)sp * (dv + 2) + dv]);
    float L = 0.f;
    for (int sp = 0; sp < splits; ++sp) {
      const float m = src[(long)sp * (dv + 2) + dv];
      const float w = m == -INFINITY ? 0.f : expf(m - M);
      wgt[sp] = w;
      L += src[(long)sp * (dv + 2) + dv + 1] * w;
    }
    inv_l = 1.f / L;
  }
  __syncthreads();
  bf16* orow = out + (long)cu_seqlens[b] * os_t + (long)head * os_h;
  for (int n = threadIdx.x; n < dv; n += blockDim.x) {
    float acc = 0.f;
    for (int sp = 0; sp < splits; ++sp)
      if (wgt[sp] != 0.f) acc = fmaf(src[(long)sp * (dv + 2) + n], wgt[sp], acc);
    orow[n] = __float2bfloat16_rn(acc * inv_l);
  }
}

template <int NT>
static int launch_latent_tc(const bf16* q, long qs_t, long qs_h, const bf16* pages, int dk, int dv,
                            const int* block_table, int max_pages, const int* cu_seqlens, const int* kv_lens,
                            const float* sink, bf16* out, long os_t, long os_h, int num_seqs, int max_query_len, int H,
                            int ps, float scale, int window, int splits, float* part, cudaStream_t stream) {
  int hgp = 1;
  while (hgp < H && hgp < LTC_BM) hgp <<= 1;
  const int tq = LTC_BM / hgp;
  const size_t rest = (size_t)LTC_BM * (dk + 8) * sizeof(bf16) + (size_t)LTC_BM * LTC_SS * sizeof(float) +
                      (size_t)LTC_BM * LTC_PS * sizeof(bf16) + 3 * LTC_BM * sizeof(float);
  const size_t tile = (size_t)LTC_BN * (dk + 8) * sizeof(bf16);
  const int stages = rest + 2 * tile <= 220 * 1024 ? 2 : 1;
  const size_t smem = rest + stages * tile;
  if (smem > 220 * 1024) return Q3_ERR_UNSUPPORTED;
  static bool configured[Q3_MAX_DEVICES] = {};
  const int device = q3_current_device();
  if (!configured[device]) {
    if (cudaFuncSetAttribute(latent_attention_tc_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             220 * 1024) != cudaSuccess)
      return Q3_ERR_LAUNCH;
    configured[device] = true;
  }
  const dim3 grid(splits > 1 ? splits : (max_query_len + tq - 1) / tq, (H + hgp - 1) / hgp, num_seqs);
  if (grid.y > 65535 || grid.z > 65535) return Q3_ERR_UNSUPPORTED;
  if (launch_pdl(latent_attention_tc_kernel<NT>, grid, dim3(LTC_THREADS), smem, stream, q, qs_t, qs_h, pages, dk, dv,
                 block_table, max_pages, cu_seqlens, kv_lens, sink, out, os_t, os_h, H, hgp, ps, scale, window,
                 splits, part, stages) != cudaSuccess)
    return Q3_ERR_LAUNCH;
  if (splits > 1 &&
      launch_pdl(latent_attention_merge_kernel, dim3(num_seqs * H), dim3(128), 0, stream, (const float*)part,
                 cu_seqlens, out, os_t, os_h, H, dv, splits) != cudaSuccess)
    return Q3_ERR_LAUNCH;
  return Q3_OK;
}

// bfloat16 only.  q: (t, h, d) at q + t*qs_t + h*qs_h + d with 16-byte aligned rows (strides multiples
// of 8); pages: [num_pages, ps, dk] dense; dk and dv multiples of 16, dv <= dk, dv <= 512.  Sequence b
// brings the packed tokens cu_seqlens[b] .. cu_seqlens[b + 1] - 1, the last of them at position
// kv_lens[b] - 1; max_query_len bounds the tokens of one sequence.  Returns Q3_ERR_UNSUPPORTED for
// other sizes (the general kernel takes those).  splits > 1 (at most 64, only with max_query_len 1):
// every sequence's keys in that many slices, part: fp32 scratch of num_seqs * H * splits * (dv + 2).
Q3_EXPORT int q3_latent_attention_tc(const void* q, long qs_t, long qs_h, const void* pages, int dk, int dv,
                                     const int* block_table, int max_pages, const int* cu_seqlens,
                                     const int* kv_lens, const float* sink, void* out, long os_t, long os_h,
                                     int num_seqs, int max_query_len, int H, int ps, float scale, int window,
                                     int splits, float* part, cudaStream_t stream) {
  if (splits < 1 || splits > 64 || (splits > 1 && (max_query_len != 1 || !part))) return Q3_ERR_ARGUMENT;
  if (!q || !pages || !block_table || !cu_seqlens || !kv_lens || !out) return Q3_ERR_ARGUMENT;
  if (H < 1 || ps < 1 || dk < 16 || dv < 16 || dv > dk) return Q3_ERR_ARGUMENT;
  if (dk % 16 || dv % 16 || dv > 512 || qs_t % 8 || qs_h % 8 || os_t % 2 || os_h % 2) return Q3_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(pages) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 3))
    return Q3_ERR_UNSUPPORTED;
  if (num_seqs == 0 || max_query_len == 0) return Q3_OK;
#define LTC_GO(NT)                                                                                                   \
  return launch_latent_tc<NT>((const bf16*)q, qs_t, qs_h, (const bf16*)pages, dk, dv, block_table, max_pages,         \
                              cu_seqlens, kv_lens, sink, (bf16*)out, os_t, os_h, num_seqs, max_query_len, H, ps, scale, \
                              window, splits, part, stream)
  if (dv <= 64) LTC_GO(2);
  if (dv <= 128) LTC_GO(4);
  if (dv <= 256) LTC_GO(8);
  LTC_GO(16);
#undef LTC_GO
}
