// Attention over a low-rank latent that all heads share (multi-head latent attention), with a sink.
//
// A token's cache row is [c | kr]: the RMS-normed latent c (R values) and one rotated key part kr (r values) that every
// head uses.  Head h has its own up-projections: key_h = U_h c (dn values) and value_h = V_h c (dv values).  The score of
// query (qn_h | qr_h) against a token is (qn_h . U_h c + qr_h . kr) * scale, and since qn_h . U_h c = (U_h^T qn_h) . c
// the keys are never built: the query is carried into the latent space once per row and head (qa_h = U_h^T qn_h, a
// product over heads, tlc_linear_heads), every head then attends over the SAME rows [c | kr] with the query
// [qa_h | qr_h], the values are the rows' first R columns, and the head's output sum_j p_j c_j goes through V_h
// afterwards (tlc_linear_heads again).  So the cache is read once for all heads, and a layer that borrows another
// layer's latents needs nothing but its own U and V.
//
// The softmax has a sink: a learned logit per head that takes part in the maximum and the denominator only (it is not
// scaled, has no value, and counts once).  Scores, softmax statistics, rotation angles, the norm of c and all
// accumulators are 32-bit.  The rotation is the interleaved one: dimensions (2i, 2i+1) of the first `rot` dimensions
// turn by position * inv_freq[i]; what lies beyond passes unchanged.
#include "common.cuh"

// ---- per row: rotate, norm, store ---------------------------------------------------------------------
// proj [T, ld] float: the row's queries at q_off, H heads of (dn | r); its down-projection (R | r) at dkv_off, or
// dkv_off < 0 for a layer that reads another layer's rows.  Writes qn [T, H*dn] (the unrotated query parts), the
// rotated parts into the last r columns of every head of qa [T, H*(R+r)], and, with a down-projection, the cache row.
template <typename TC>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const float* __restrict__ proj, int ld, int q_off, int dkv_off, const float* __restrict__ cw, float eps,
                      const float* __restrict__ inv_freq, int rot, const int* __restrict__ positions,
                      const int* __restrict__ row_seq, const int* __restrict__ slots, const int* __restrict__ block_table,
                      int max_pages, TC* __restrict__ pages, TC* __restrict__ qn, TC* __restrict__ qa, int H, int dn, int r,
                      int R) {
  tlc_pdl(proj, pages, qn, qa);
  __shared__ float red[33];
  const int t = blockIdx.x;
  const float* pr = proj + (size_t)t * ld;
  const int pos = positions[t];
  const float fpos = (float)pos;
  const int hw = dn + r, aw = R + r;
  for (int i = threadIdx.x; i < H * dn; i += blockDim.x) {
    const int h = i / dn, d = i - h * dn;
    qn[(size_t)t * H * dn + i] = from_f32<TC>(pr[q_off + h * hw + d]);
  }
  // rotated parts: pairs of the first `rot` dimensions, single dimensions beyond
  const int half = rot >> 1, per = half + (r - rot);
  for (int i = threadIdx.x; i < H * per; i += blockDim.x) {
    const int h = i / per, j = i - h * per;
    const float* src = pr + q_off + h * hw + dn;
    TC* dst = qa + (size_t)t * H * aw + (size_t)h * aw + R;
    if (j < half) {
      float sn, cs;
      sincosf(fpos * inv_freq[j], &sn, &cs);
      const float u = src[2 * j], v = src[2 * j + 1];
      dst[2 * j] = from_f32<TC>(u * cs - v * sn);
      dst[2 * j + 1] = from_f32<TC>(v * cs + u * sn);
    } else {
      const int d = rot + (j - half);
      dst[d] = from_f32<TC>(src[d]);
    }
  }
  if (dkv_off < 0) return;
  const float* cr = pr + dkv_off;
  float ss = 0.f;
  for (int d = threadIdx.x; d < R; d += blockDim.x) { const float v = cr[d]; ss += v * v; }
  ss = block_sum(ss, red);
  const float s = 1.0f / sqrtf(ss / (float)R + eps);
  const int page = block_table[(size_t)slots[row_seq[t]] * max_pages + pos / TLC_PAGE];
  TC* row = pages + ((size_t)page * TLC_PAGE + pos % TLC_PAGE) * aw;
  for (int d = threadIdx.x; d < R; d += blockDim.x) row[d] = from_f32<TC>(cr[d] * s * cw[d]);
  for (int j = threadIdx.x; j < per; j += blockDim.x) {
    const float* src = cr + R;
    if (j < half) {
      float sn, cs;
      sincosf(fpos * inv_freq[j], &sn, &cs);
      const float u = src[2 * j], v = src[2 * j + 1];
      row[R + 2 * j] = from_f32<TC>(u * cs - v * sn);
      row[R + 2 * j + 1] = from_f32<TC>(v * cs + u * sn);
    } else {
      const int d = rot + (j - half);
      row[R + d] = from_f32<TC>(src[d]);
    }
  }
}

extern "C" int tlc_latent_prepare(const float* proj, int ld, int q_off, int dkv_off, const float* cw, float eps,
                                  const float* inv_freq, int rot, const int* positions, const int* row_seq, const int* slots,
                                  const int* block_table, int max_pages, void* pages, void* qn, void* qa, int dtype, int T, int H,
                                  int dn, int r, int R, cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= r, "latent_prepare: %d rotated dimensions of %d", rot, r);
  TLC_DISPATCH_DTYPE(dtype, TC, tlc_launch(latent_prepare_kernel<TC>, dim3(T), dim3(128), 0, stream, proj, ld, q_off, dkv_off, cw, eps,
                                           inv_freq, rot, positions, row_seq, slots, block_table, max_pages, (TC*)pages, (TC*)qn,
                                           (TC*)qa, H, dn, r, R));
  TLC_CHECK_LAUNCH("latent_prepare");
  return 0;
}

// ---- attention, a warp per (row, head): any sizes, both element types ------------------------------------
// qa [T, H, R+r]; pages [n_pages, 64, R+r]; out [T, H, R] = sum_j p_j c_j with p the softmax over the row's keys
// 0..position and the head's sink.  A lane scores one key of 32 at a time; the output's R columns are lane-strided.
#define LAT_MAXV 16     // R <= 32 * LAT_MAXV
template <typename TC>
__global__ void __launch_bounds__(128)
latent_attention_warp_kernel(const TC* __restrict__ qa, const TC* __restrict__ pages, const float* __restrict__ sink,
                             const int* __restrict__ block_table, int max_pages, const int* __restrict__ positions,
                             const int* __restrict__ row_seq, const int* __restrict__ slots, TC* __restrict__ out, int H, int R,
                             int r, float scale) {
  tlc_pdl(qa, pages, out);
  extern __shared__ float sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x, h = blockIdx.y * 4 + warp;
  if (h >= H) return;
  const int aw = R + r;
  float* qs = sh + (size_t)warp * aw;
  const TC* qr = qa + ((size_t)t * H + h) * aw;
  for (int d = lane; d < aw; d += 32) qs[d] = to_f32(qr[d]) * scale;
  __syncwarp();
  const int n_keys = positions[t] + 1;
  const int* table = block_table + (size_t)slots[row_seq[t]] * max_pages;
  float m = sink[h], l = 1.0f;             // the sink: exp(sink - m) with m = sink
  float acc[LAT_MAXV];
#pragma unroll
  for (int i = 0; i < LAT_MAXV; i++) acc[i] = 0.f;
  for (int k0 = 0; k0 < n_keys; k0 += 32) {
    const int kp = k0 + lane;
    float s = -INFINITY;
    if (kp < n_keys) {
      const TC* kr = pages + ((size_t)table[kp / TLC_PAGE] * TLC_PAGE + kp % TLC_PAGE) * aw;
      float dot = 0.f;
      for (int d = 0; d < aw; d++) dot = fmaf(to_f32(kr[d]), qs[d], dot);
      s = dot;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = kp < n_keys ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < LAT_MAXV; i++) acc[i] *= corr;
    const int nk = min(32, n_keys - k0);
    for (int j = 0; j < nk; j++) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int kj = k0 + j;
      const TC* vr = pages + ((size_t)table[kj / TLC_PAGE] * TLC_PAGE + kj % TLC_PAGE) * aw;
#pragma unroll
      for (int i = 0; i < LAT_MAXV; i++) {
        const int d = lane + 32 * i;
        if (d < R) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
      }
    }
    m = m_new;
  }
  const float inv = 1.0f / l;
  TC* o = out + ((size_t)t * H + h) * R;
#pragma unroll
  for (int i = 0; i < LAT_MAXV; i++) {
    const int d = lane + 32 * i;
    if (d < R) o[d] = from_f32<TC>(acc[i] * inv);
  }
}

extern "C" int tlc_latent_attention(const void* qa, const void* pages, int dtype, const float* sink, const int* block_table,
                                    int max_pages, const int* positions, const int* row_seq, const int* slots, void* out, int T,
                                    int H, int R, int r, float scale, cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(R >= 1 && R <= 32 * LAT_MAXV, "latent_attention: a latent of %d values exceeds the kernel's limit of %d", R, 32 * LAT_MAXV);
  const size_t smem = (size_t)4 * (R + r) * sizeof(float);
  TLC_REQUIRE(smem <= 48 * 1024, "latent_attention: a key row of %d values is too wide", R + r);
  dim3 grid(T, (H + 3) / 4);
  TLC_DISPATCH_DTYPE(dtype, TC, tlc_launch(latent_attention_warp_kernel<TC>, grid, dim3(128), smem, stream, (const TC*)qa,
                                           (const TC*)pages, sink, block_table, max_pages, positions, row_seq, slots, (TC*)out, H, R, r,
                                           scale));
  TLC_CHECK_LAUNCH("latent_attention");
  return 0;
}

// ---- a product per head ------------------------------------------------------------------------------------
// out[t, h, n] = sum_k a[t, h, k] * w[h, n, k]: a [T, H, K] with row stride lda and head stride a_hs, w [H, N, K] dense,
// out with row stride ldo and head stride o_hs.  Tiles of 32 rows x 32 columns, 32-bit sums on the CUDA cores.
#define LH_TM 32
#define LH_TN 32
#define LH_TK 32
template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
linear_heads_kernel(const TA* __restrict__ a, int lda, int a_hs, const TW* __restrict__ w, TO* __restrict__ out, int ldo,
                    int o_hs, int T, int N, int K) {
  tlc_pdl(a, out);
  __shared__ float As[LH_TK][LH_TM + 1], Ws[LH_TK][LH_TN + 1];
  const int h = blockIdx.z, m0 = blockIdx.x * LH_TM, n0 = blockIdx.y * LH_TN;
  const TA* ah = a + (size_t)h * a_hs;
  const TW* wh = w + (size_t)h * N * K;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;     // columns tx, tx+16; rows ty, ty+16
  float c00 = 0.f, c01 = 0.f, c10 = 0.f, c11 = 0.f;
  for (int k0 = 0; k0 < K; k0 += LH_TK) {
    for (int i = threadIdx.x; i < LH_TM * LH_TK; i += 256) {
      const int rr = i / LH_TK, kk = i % LH_TK;
      const int m = m0 + rr, k = k0 + kk;
      As[kk][rr] = (m < T && k < K) ? to_f32(ah[(size_t)m * lda + k]) : 0.f;
      const int n = n0 + rr;
      Ws[kk][rr] = (n < N && k < K) ? to_f32(wh[(size_t)n * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < LH_TK; kk++) {
      const float a0 = As[kk][ty], a1 = As[kk][ty + 16], w0 = Ws[kk][tx], w1 = Ws[kk][tx + 16];
      c00 = fmaf(a0, w0, c00); c01 = fmaf(a0, w1, c01);
      c10 = fmaf(a1, w0, c10); c11 = fmaf(a1, w1, c11);
    }
    __syncthreads();
  }
  TO* oh = out + (size_t)h * o_hs;
  const int ma = m0 + ty, mb = m0 + ty + 16, na = n0 + tx, nb = n0 + tx + 16;
  if (ma < T && na < N) oh[(size_t)ma * ldo + na] = from_f32<TO>(c00);
  if (ma < T && nb < N) oh[(size_t)ma * ldo + nb] = from_f32<TO>(c01);
  if (mb < T && na < N) oh[(size_t)mb * ldo + na] = from_f32<TO>(c10);
  if (mb < T && nb < N) oh[(size_t)mb * ldo + nb] = from_f32<TO>(c11);
}

extern "C" int tlc_linear_heads(const void* a, int a_dtype, int lda, int a_hs, const void* w, int w_dtype, void* out,
                                int out_dtype, int ldo, int o_hs, int T, int H, int N, int K, cudaStream_t stream) {
  if (T == 0 || H == 0 || N == 0) return 0;
  TLC_REQUIRE(K > 0 && H <= 65535, "linear_heads: bad sizes H=%d K=%d", H, K);
  dim3 grid((T + LH_TM - 1) / LH_TM, (N + LH_TN - 1) / LH_TN, H);
  TLC_DISPATCH_DTYPE(a_dtype, TA, TLC_DISPATCH_DTYPE(w_dtype, TW, TLC_DISPATCH_DTYPE(out_dtype, TO,
      tlc_launch(linear_heads_kernel<TA, TW, TO>, grid, dim3(256), 0, stream, (const TA*)a, lda, a_hs, (const TW*)w, (TO*)out, ldo,
                 o_hs, T, N, K))));
  TLC_CHECK_LAUNCH("linear_heads");
  return 0;
}
