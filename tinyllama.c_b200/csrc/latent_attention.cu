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
// The softmax has a sink: a per-head logit, used as stored (the score scale does not apply to it), that adds a single
// term to the denominator and nothing to the weighted sum of values.  Scores, softmax statistics, rotation angles, the norm of c and all
// accumulators are 32-bit.  The rotation is the interleaved one: dimensions (2i, 2i+1) of the first `rot` dimensions
// turn by position * inv_freq[i]; what lies beyond passes unchanged.
#include "common.cuh"

// ---- per row: rotate, norm, store ---------------------------------------------------------------------
// qproj [T, ldq] float: the row's queries at q_off, H heads of (dn | r); proj [T, ld] float: its down-projection (R | r)
// at dkv_off, or dkv_off < 0 for a layer that reads another layer's rows (the two may be one buffer).  Writes qn [T, H*dn] (the unrotated query parts), the
// rotated parts into the last r columns of every head of qa [T, H*(R+r)], and, with a down-projection, the cache row.
template <typename TC>
__global__ void __launch_bounds__(512)
latent_prepare_kernel(const float* __restrict__ qproj, int ldq, int q_off, const float* __restrict__ proj, int ld, int dkv_off,
                      const float* __restrict__ cw, float eps,
                      const float* __restrict__ inv_freq, int rot, const int* __restrict__ positions,
                      const int* __restrict__ row_seq, const int* __restrict__ slots, const int* __restrict__ block_table,
                      int max_pages, TC* __restrict__ pages, TC* __restrict__ qn, TC* __restrict__ qa, int H, int dn, int r,
                      int R) {
  tlc_pdl(qproj, proj, pages, qn, qa);
  __shared__ float red[33];
  const int t = blockIdx.x;
  const float* pr = qproj + (size_t)t * ldq;
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
  const float* cr = proj + (size_t)t * ld + dkv_off;
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

extern "C" int tlc_latent_prepare(const float* qproj, int ldq, int q_off, const float* proj, int ld, int dkv_off, const float* cw,
                                  float eps,
                                  const float* inv_freq, int rot, const int* positions, const int* row_seq, const int* slots,
                                  const int* block_table, int max_pages, void* pages, void* qn, void* qa, int dtype, int T, int H,
                                  int dn, int r, int R, cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= r, "latent_prepare: %d rotated dimensions of %d", rot, r);
  const int nt = T < 256 ? 512 : 128;                       // few rows: more threads a row
  TLC_DISPATCH_DTYPE(dtype, TC, tlc_launch(latent_prepare_kernel<TC>, dim3(T), dim3(nt), 0, stream, qproj, ldq, q_off, proj, ld, dkv_off, cw, eps,
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
                             int r, float scale, int window) {
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
  float m = -INFINITY, l = 0.f;
  if (sink) { m = sink[h]; l = 1.0f; }     // the sink: exp(sink - m) with m = sink
  const int k_first = window > 0 ? max(0, n_keys - window) : 0;     // a window: the last `window` keys
  float acc[LAT_MAXV];
#pragma unroll
  for (int i = 0; i < LAT_MAXV; i++) acc[i] = 0.f;
  for (int k0 = k_first; k0 < n_keys; k0 += 32) {
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
                                    int H, int R, int r, float scale, int window, cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(R >= 1 && R <= 32 * LAT_MAXV, "latent_attention: a latent of %d values exceeds the kernel's limit of %d", R, 32 * LAT_MAXV);
  const size_t smem = (size_t)4 * (R + r) * sizeof(float);
  TLC_REQUIRE(smem <= 48 * 1024, "latent_attention: a key row of %d values is too wide", R + r);
  dim3 grid(T, (H + 3) / 4);
  TLC_DISPATCH_DTYPE(dtype, TC, tlc_launch(latent_attention_warp_kernel<TC>, grid, dim3(128), smem, stream, (const TC*)qa,
                                           (const TC*)pages, sink, block_table, max_pages, positions, row_seq, slots, (TC*)out, H, R, r,
                                           scale, window));
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

// ---- attention on the tensor cores (bfloat16 rows) -----------------------------------------------------------------
// All heads of a row attend over the same cached rows, so (row, head) pairs are the M side of one product: a block takes
// a tile of 64 pairs of ONE sequence -- HP heads (a power of two, H padded up to it, at most 64) of 64 / HP consecutive
// rows -- and walks the sequence's pages.  A page [64 keys, R + r] arrives by cp.async (two in flight) and serves twice:
// as the keys of S = Q K^T (all R + r columns) and as the values of O += P V (its first R columns, read transposed by
// ldmatrix), so the cache is read once for both and once for all heads.  Four warps of 16 pairs each; scores, running
// maximum and sum and the output accumulator are 32-bit registers, the softmax numerators that multiply the values are
// bfloat16.  The key range of a tile may be cut into n_split ranges that run as blocks of their own (single-token steps,
// pieces of long prompts) and leave (maximum, sum, unnormalised output) in 32-bit scratch; the merge adds them up and
// brings in the head's sink, which enters the maximum and the denominator only.  With one range the block finishes the
// rows itself.
#define LT_M 64
#define LT_KEYS TLC_PAGE
__device__ __forceinline__ void lt_cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void lt_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void lt_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void lt_ldsm4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void lt_ldsm4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void lt_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lt_pack(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// MAXNV: pairs of 8-column tiles of the output a thread may hold (R <= 16 * MAXNV).  NWARP: warps of 16 pairs each; a
// prompt's tiles take 8 (128 pairs share every page that arrives), single-token steps 4.
template <int MAXNV, int NWARP>
__global__ void __launch_bounds__(NWARP * 32)
latent_attention_tc_kernel(const __nv_bfloat16* __restrict__ qa, const __nv_bfloat16* __restrict__ pages,
                           const float* __restrict__ sink, const int* __restrict__ block_table, int max_pages,
                           const int* __restrict__ cu_seqlens, const int* __restrict__ slots, const int* __restrict__ start_pos,
                           __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, int B, int H,
                           int HP, int R, int r, float scale, int n_split, int n_tiles, int window) {
  tlc_pdl(qa, pages, out, part_o, part_ml);
  constexpr int LTM = NWARP * 16, NT = NWARP * 32;
  extern __shared__ __align__(16) unsigned char lt_smem[];
  const int aw = R + r, ldsm = aw + 8;                    // padded row: ldmatrix rows land in different banks
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(lt_smem);
  __nv_bfloat16* ks = qs + (size_t)LTM * ldsm;           // two buffers of [64][ldsm]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, q4 = lane & 3;
  const int rpt = LTM / HP, n_hg = (H + HP - 1) / HP;    // rows per tile, head groups
  // which sequence, rows and heads this tile covers
  // the last rows of a sequence see the most keys: the grid starts with the highest tiles, so that the longest blocks
  // run first and the short ones fill the tail
  int tile = blockIdx.x / n_hg;
  const int hg = blockIdx.x - tile * n_hg;
  tile = n_tiles - 1 - tile;
  int b = 0, first = 0, len = 0;
  for (; b < B; b++) {
    first = cu_seqlens[b];
    len = cu_seqlens[b + 1] - first;
    const int nt = (len + rpt - 1) / rpt;
    if (tile < nt) break;
    tile -= nt;
  }
  if (b >= B) return;
  const int row0 = tile * rpt, rows = min(rpt, len - row0);
  const int t0 = first + row0, p0 = start_pos[b] + row0;  // first packed row and its position
  const int h0 = hg * HP;
  const int n_kt_all = (p0 + rows - 1) / LT_KEYS + 1;     // key tiles the tile's last row sees
  const int kt_lo = window > 0 ? max(0, p0 - window + 1) / LT_KEYS : 0;   // the first key tile the tile's first row sees
  const int split = blockIdx.y;
  const int per = (n_kt_all - kt_lo + n_split - 1) / n_split;
  const int kt0 = kt_lo + split * per, kt1 = min(n_kt_all, kt0 + per);
  const int* table = block_table + (size_t)slots[b] * max_pages;
  const uint32_t qs_u = (uint32_t)__cvta_generic_to_shared(qs), ks_u = (uint32_t)__cvta_generic_to_shared(ks);
  const int chunks_row = aw >> 3;

  auto load_keys = [&](int kt, int buf) {
    const __nv_bfloat16* src = pages + (size_t)table[kt] * LT_KEYS * aw;
    const uint32_t dst = ks_u + (uint32_t)buf * LT_KEYS * ldsm * 2;
    for (int c = tid; c < LT_KEYS * chunks_row; c += NT) {
      const int rr = c / chunks_row, cc = c - rr * chunks_row;
      lt_cp_async16(dst + (uint32_t)(rr * ldsm + cc * 8) * 2, src + (size_t)rr * aw + cc * 8);
    }
  };
  if (kt0 < kt1) {
    // the tile's queries: pair m = row * HP + head; rows past the sequence and heads past H are zero
    for (int c = tid; c < LTM * chunks_row; c += NT) {
      const int m = c / chunks_row, cc = c - m * chunks_row;
      const int rl = m / HP, h = h0 + (m - rl * HP);
      if (rl < rows && h < H)
        lt_cp_async16(qs_u + (uint32_t)(m * ldsm + cc * 8) * 2, qa + ((size_t)(t0 + rl) * H + h) * aw + cc * 8);
      else
        *reinterpret_cast<uint4*>(qs + (size_t)m * ldsm + cc * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
    load_keys(kt0, 0);
  }
  lt_cp_commit();

  const int nv = R >> 4;                                  // pairs of output tiles in use
  float o[MAXNV][2][4];
#pragma unroll
  for (int i = 0; i < MAXNV; i++)
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) o[i][j][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int ma = warp * 16 + g, mb = ma + 8;              // this thread's two pairs
  const int pos_a = p0 + ma / HP, pos_b = p0 + mb / HP;   // their positions (keys 0..pos are visible, or the last `window`)
  const int lo_a = window > 0 ? pos_a - window + 1 : 0, lo_b = window > 0 ? pos_b - window + 1 : 0;
  const float LOG2E = 1.4426950408889634f;

  for (int kt = kt0; kt < kt1; kt++) {
    const int buf = (kt - kt0) & 1;
    if (kt + 1 < kt1) load_keys(kt + 1, buf ^ 1);
    lt_cp_commit();
    lt_cp_wait<1>();
    __syncthreads();
    const uint32_t kb = ks_u + (uint32_t)buf * LT_KEYS * ldsm * 2;
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) s[j][e] = 0.f;
    for (int k0 = 0; k0 < aw; k0 += 16) {
      uint32_t a0, a1, a2, a3;
      lt_ldsm4(a0, a1, a2, a3, qs_u + (uint32_t)((warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldsm + k0 + (lane >> 4) * 8) * 2);
#pragma unroll
      for (int jp = 0; jp < 4; jp++) {
        uint32_t b0, b1, b2, b3;
        lt_ldsm4(b0, b1, b2, b3, kb + (uint32_t)((jp * 16 + (lane & 7) + (lane >> 4) * 8) * ldsm + k0 + ((lane >> 3) & 1) * 8) * 2);
        lt_mma(s[2 * jp], a0, a1, a2, a3, b0, b1);
        lt_mma(s[2 * jp + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    // mask, scale, running maximum
    const int key0 = kt * LT_KEYS + 2 * q4;
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int k = key0 + 8 * j;
      s[j][0] = (k <= pos_a && k >= lo_a) ? s[j][0] * scale : -INFINITY;
      s[j][1] = (k + 1 <= pos_a && k + 1 >= lo_a) ? s[j][1] * scale : -INFINITY;
      s[j][2] = (k <= pos_b && k >= lo_b) ? s[j][2] * scale : -INFINITY;
      s[j][3] = (k + 1 <= pos_b && k + 1 >= lo_b) ? s[j][3] * scale : -INFINITY;
      mx_a = fmaxf(mx_a, fmaxf(s[j][0], s[j][1]));
      mx_b = fmaxf(mx_b, fmaxf(s[j][2], s[j][3]));
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_run[0], mx_a), mn_b = fmaxf(m_run[1], mx_b);
    const float ref_a = mn_a == -INFINITY ? 0.f : mn_a, ref_b = mn_b == -INFINITY ? 0.f : mn_b;
    const float ca = exp2f((m_run[0] - ref_a) * LOG2E), cb = exp2f((m_run[1] - ref_b) * LOG2E);   // exp(-inf) = 0 at first
    m_run[0] = mn_a;
    m_run[1] = mn_b;
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      s[j][0] = exp2f((s[j][0] - ref_a) * LOG2E);
      s[j][1] = exp2f((s[j][1] - ref_a) * LOG2E);
      s[j][2] = exp2f((s[j][2] - ref_b) * LOG2E);
      s[j][3] = exp2f((s[j][3] - ref_b) * LOG2E);
      sa += s[j][0] + s[j][1];
      sb += s[j][2] + s[j][3];
    }
    l_run[0] = l_run[0] * ca + sa;                        // (a thread's share; the quad's shares are added at the end)
    l_run[1] = l_run[1] * cb + sb;
#pragma unroll
    for (int i = 0; i < MAXNV; i++)
      if (i < nv) {
#pragma unroll
        for (int j = 0; j < 2; j++) { o[i][j][0] *= ca; o[i][j][1] *= ca; o[i][j][2] *= cb; o[i][j][3] *= cb; }
      }
    // O += P V: the numerators as bfloat16 A fragments, the page's first R columns as B
#pragma unroll
    for (int kk = 0; kk < 4; kk++) {
      const uint32_t a0 = lt_pack(s[2 * kk][0], s[2 * kk][1]), a1 = lt_pack(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t a2 = lt_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = lt_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int i = 0; i < MAXNV; i++)
        if (i < nv) {
          uint32_t b0, b1, b2, b3;
          lt_ldsm4_t(b0, b1, b2, b3, kb + (uint32_t)((kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldsm + i * 16 + (lane >> 4) * 8) * 2);
          lt_mma(o[i][0], a0, a1, a2, a3, b0, b1);
          lt_mma(o[i][1], a0, a1, a2, a3, b2, b3);
        }
    }
    __syncthreads();                                       // the buffer is free for the tile after the next
  }
  lt_cp_wait<0>();
  // the quad's shares of the sums
#pragma unroll
  for (int e = 0; e < 2; e++) {
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 1);
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 2);
  }
#pragma unroll
  for (int e = 0; e < 2; e++) {
    const int m = e == 0 ? ma : mb;
    const int rl = m / HP, h = h0 + (m - rl * HP);
    if (rl >= rows || h >= H) continue;
    const size_t th = (size_t)(t0 + rl) * H + h;
    if (n_split > 1) {
      float* po = part_o + (th * n_split + split) * R;
      if (q4 == 0) {
        part_ml[(th * n_split + split) * 2] = m_run[e];
        part_ml[(th * n_split + split) * 2 + 1] = l_run[e];
      }
#pragma unroll
      for (int i = 0; i < MAXNV; i++)
        if (i < nv) {
#pragma unroll
          for (int j = 0; j < 2; j++)
            *reinterpret_cast<float2*>(po + i * 16 + j * 8 + 2 * q4) = make_float2(o[i][j][2 * e], o[i][j][2 * e + 1]);
        }
    } else {
      const float sk = sink ? sink[h] : -INFINITY;         // no sink: nothing joins the denominator
      const float mf = fmaxf(m_run[e], sk);
      const float w = exp2f((m_run[e] - mf) * LOG2E);
      const float inv = w / (l_run[e] * w + exp2f((sk - mf) * LOG2E));
      __nv_bfloat16* po = out + th * R;
#pragma unroll
      for (int i = 0; i < MAXNV; i++)
        if (i < nv) {
#pragma unroll
          for (int j = 0; j < 2; j++)
            *reinterpret_cast<uint32_t*>(po + i * 16 + j * 8 + 2 * q4) = lt_pack(o[i][j][2 * e] * inv, o[i][j][2 * e + 1] * inv);
        }
    }
  }
}

// out[t, h, :] from the ranges' (maximum, sum, unnormalised output) and the head's sink.  A block per (row, head); a
// thread per output column, all ranges' loads of a column in flight together.
__global__ void __launch_bounds__(128)
latent_attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const float* __restrict__ sink,
                              __nv_bfloat16* __restrict__ out, int H, int R, int n_split) {
  tlc_pdl(part_o, part_ml, out);
  __shared__ float wsh[64];
  const int th = blockIdx.x;
  const float sk = sink ? sink[th % H] : -INFINITY;
  const float* ml = part_ml + (size_t)th * n_split * 2;
  float mf = sk;
  for (int s = 0; s < n_split; s++) mf = fmaxf(mf, ml[2 * s]);
  float den = expf(sk - mf);
  for (int s = 0; s < n_split; s++) den += ml[2 * s + 1] * expf(ml[2 * s] - mf);     // an empty range: sum 0, exp(-inf) = 0
  const float inv = 1.0f / den;
  if (threadIdx.x < n_split) wsh[threadIdx.x] = expf(ml[2 * threadIdx.x] - mf) * inv;
  __syncthreads();
  for (int d = threadIdx.x; d < R; d += blockDim.x) {
    float acc = 0.f;
#pragma unroll 8
    for (int s = 0; s < n_split; s++) {
      const float w = wsh[s];
      const float v = part_o[((size_t)th * n_split + s) * R + d];
      acc = w > 0.f ? fmaf(v, w, acc) : acc;
    }
    out[(size_t)th * R + d] = __float2bfloat16_rn(acc);
  }
}

static int g_lt_smem_set = 0;
extern "C" int tlc_latent_attention_tc_ok(int dtype, int H, int R, int r) {
  if (dtype != TLC_BF16 || R % 16 || (R + r) % 16 || R > 256 || H < 1) return 0;
  const size_t smem = (size_t)3 * LT_M * (R + r + 8) * 2;
  return smem <= 200 * 1024 ? 1 : 0;
}

// How many (row, head) pairs a tile takes: 128 for steps that bring several rows a sequence (where shared memory holds
// such a tile beside two pages), else 64.
extern "C" int tlc_latent_attention_tc_tile(int T, int B, int R, int r) {
  const size_t smem = (size_t)(128 + 2 * LT_KEYS) * (R + r + 8) * 2;
  return (T >= 4 * B && smem <= 200 * 1024) ? 128 : 64;
}

// How many ranges the keys of a tile are cut into: none while the tiles fill the GPU, else as many as bring the grid
// to about two blocks an SM, at most one per page.
extern "C" int tlc_latent_attention_tc_splits(int n_tiles, int max_keys) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int pages = (max_keys + LT_KEYS - 1) / LT_KEYS;
  if (n_tiles >= sms || pages <= 1) return 1;
  int s = (2 * sms + n_tiles - 1) / n_tiles;
  if (s > pages) s = pages;
  if (s > 64) s = 64;
  return s < 1 ? 1 : s;
}

extern "C" int tlc_latent_attention_tc(const void* qa, const void* pages, const float* sink, const int* block_table, int max_pages,
                                       const int* cu_seqlens, const int* slots, const int* start_pos, void* out, float* part_o,
                                       float* part_ml, int B, int T, int tile_pairs, int n_tiles, int H, int R, int r, float scale,
                                       int n_split, int window, cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(tlc_latent_attention_tc_ok(TLC_BF16, H, R, r), "latent_attention_tc: sizes H=%d R=%d r=%d are not built", H, R, r);
  TLC_REQUIRE(n_split >= 1 && n_split <= 64 && (n_split == 1 || (part_o && part_ml)), "latent_attention_tc: %d key ranges (1..64; more than one needs scratch)", n_split);
  TLC_REQUIRE(tile_pairs == 64 || (tile_pairs == 128 && tlc_latent_attention_tc_tile(1 << 20, 1, R, r) == 128),
              "latent_attention_tc: tiles of %d pairs are not built for R=%d r=%d", tile_pairs, R, r);
  int HP = 1;
  while (HP < H && HP < 64) HP <<= 1;
  const int n_hg = (H + HP - 1) / HP;
  const size_t smem = (size_t)(tile_pairs + 2 * LT_KEYS) * (R + r + 8) * 2;
  if (!g_lt_smem_set) {
    cudaFuncSetAttribute(latent_attention_tc_kernel<8, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(latent_attention_tc_kernel<16, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(latent_attention_tc_kernel<8, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(latent_attention_tc_kernel<16, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    g_lt_smem_set = 1;
  }
  dim3 grid(n_tiles * n_hg, n_split);
  typedef const __nv_bfloat16* BP;
#define LT_LAUNCH(NV, NW)                                                                                                      \
  tlc_launch(latent_attention_tc_kernel<NV, NW>, grid, dim3(NW * 32), smem, stream, (BP)qa, (BP)pages, sink, block_table, max_pages, \
             cu_seqlens, slots, start_pos, (__nv_bfloat16*)out, part_o, part_ml, B, H, HP, R, r, scale, n_split, n_tiles, window)
  if (tile_pairs == 128) { if (R <= 128) LT_LAUNCH(8, 8); else LT_LAUNCH(16, 8); }
  else { if (R <= 128) LT_LAUNCH(8, 4); else LT_LAUNCH(16, 4); }
#undef LT_LAUNCH
  TLC_CHECK_LAUNCH("latent_attention_tc");
  if (n_split > 1) {
    tlc_launch(latent_attention_merge_kernel, dim3(T * H), dim3(128), 0, stream, (const float*)part_o, (const float*)part_ml, sink,
               (__nv_bfloat16*)out, H, R, n_split);
    TLC_CHECK_LAUNCH("latent_attention_merge");
  }
  return 0;
}
