// Attention of prompt portions over the paged cache on warp tensor-core instructions, with the mask, the sink and the
// gate of attention_masked.cu (the same visibility rule; see there). bfloat16 queries, keys and values.
//
// A CTA of four warps owns 64 consecutive rows of one request and one head; a warp owns 16 of the rows. Keys go by in
// tiles of 64 ABSOLUTE positions, from the first tile any of the CTA's rows sees to the tile of its last row (for a
// window that keeps the first tokens: those tiles first), gathered row by row into shared memory with cp.async (16
// bytes a copy, the next tile while this one is worked on; a key no row of the CTA sees, or whose page was given back,
// is zero-filled and never read). S = Q K^T and O += P V are mma.sync m16n8k16 with 32-bit accumulators; the scale, the
// mask, the running maximum and sums and exp are 32-bit (the online softmax of one pass); P is rounded to bfloat16 for
// the second product. The sink joins the denominator at the end; the gate multiplies the result; one rounding on the
// way out. Keys and values are addressed by (page, head, offset) strides, so the same kernel reads the paged planes
// ([page][G][page_size][width]) and a token-major buffer of keys and values made for one request (page_size 1).
//
// Sizes are template parameters (D = 16 DK, E = 8 EN) because the accumulators live in registers; a size that is not
// instantiated is refused by hb_attn_masked_flash_supported and goes to the row kernel.
#include "common.cuh"

struct FlashMaskedArgs {
  const __nv_bfloat16* q; long ldq;
  const __nv_bfloat16* kc; long k_page, k_head, k_row;
  const __nv_bfloat16* vc; long v_page, v_head, v_row;
  const int* bt; int bt_stride;
  const int* q_start; const int* q_len; const int* ctx_len; int req0;
  int row_limit;                        // requests that bring fewer rows are left to the row kernel
  const float* sink;
  const float* gate; long ld_gate; int gate_off; int gate_mode;
  void* out; long ldo;
  int H, G, page_size, mask, window, keep_first, chunk;
  float scale;
};

__device__ __forceinline__ void fm_cp16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void fm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void fm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fm_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t fm_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}
__device__ __forceinline__ void fm_lo_keep(const FlashMaskedArgs& A, int p, int& lo, int& keep) {
  lo = 0;
  keep = 0;
  if (A.mask == 1 && A.window > 0) {
    lo = max(0, p - A.window + 1);
    keep = min(A.keep_first, p + 1);
  } else if (A.mask == 2 && A.chunk > 0) {
    lo = (p / A.chunk) * A.chunk;
  }
}

constexpr int FM_ROWS = 64, FM_KEYS = 64, FM_THREADS = 128;

template <int DK, int EN, typename TO>
__global__ void __launch_bounds__(FM_THREADS) attn_masked_flash_kernel(FlashMaskedArgs A) {
  constexpr int D = 16 * DK, E = 8 * EN, KP = D + 8, VP = E + 8;      // padded rows: consecutive keys fall on different banks
  extern __shared__ __align__(16) uint8_t fm_smem[];
  __nv_bfloat16* Ks = (__nv_bfloat16*)fm_smem;                        // [2][FM_KEYS][KP]
  __nv_bfloat16* Vs = Ks + 2 * FM_KEYS * KP;                          // [2][FM_KEYS][VP]
  hb_pdl_launch();
  hb_pdl_wait();
  const int r = A.req0 + blockIdx.z, h = blockIdx.y, qt = blockIdx.x;
  const int qlen = A.q_len[r];
  if (qlen < A.row_limit || qt * FM_ROWS >= qlen) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, quad = lane >> 2, qi = lane & 3;
  const int rows = min(FM_ROWS, qlen - qt * FM_ROWS), t0 = A.q_start[r] + qt * FM_ROWS, p0 = A.ctx_len[r] + qt * FM_ROWS;
  const int p_last = p0 + rows - 1, g = h / (A.H / A.G), ps = A.page_size;
  const int* table = A.bt + (size_t)r * A.bt_stride;
  // the tiles the CTA walks: those of the kept first tokens, then from the first row's look-back to the last row
  int lo_first, keep_first_row, lo_tmp, keep_last;
  fm_lo_keep(A, p0, lo_first, keep_first_row);
  fm_lo_keep(A, p_last, lo_tmp, keep_last);
  const int last_keep_tile = keep_last > 0 ? (keep_last - 1) / FM_KEYS : -1;
  const int first_win_tile = max(lo_first / FM_KEYS, last_keep_tile + 1);
  const int n_tiles = (last_keep_tile + 1) + (p_last / FM_KEYS - first_win_tile + 1);
  auto tile_at = [&](int i) { return i <= last_keep_tile ? i : first_win_tile + (i - (last_keep_tile + 1)); };

  // Where a tile's 64 keys lie (element offsets of their key and value rows, -1: not wanted or its page given back) is
  // looked up once a tile, by one thread a key, a tile before the copies that use it are issued: the copies themselves
  // then wait for no load.
  __shared__ long kofs[2][FM_KEYS], vofs[2][FM_KEYS];
  auto locate = [&](int slot, int tile) {
    if (tid < FM_KEYS) {
      const int kp = tile * FM_KEYS + tid;
      const bool want = kp <= p_last && (kp >= lo_first || kp < keep_last);
      const int page = want ? table[kp / ps] : -1;
      const int off = kp % ps;
      kofs[slot][tid] = page >= 0 ? (long)page * A.k_page + (long)g * A.k_head + (long)off * A.k_row : -1;
      vofs[slot][tid] = page >= 0 ? (long)page * A.v_page + (long)g * A.v_head + (long)off * A.v_row : -1;
    }
  };
  auto load_tile = [&](int buf, int slot) {
    __nv_bfloat16* kd = Ks + buf * FM_KEYS * KP;
    __nv_bfloat16* vd = Vs + buf * FM_KEYS * VP;
    constexpr int CK = D / 8, CV = E / 8;
    for (int i = tid; i < FM_KEYS * (CK + CV); i += FM_THREADS) {
      const int kr = i / (CK + CV), c = i - kr * (CK + CV);
      __nv_bfloat16* dst = c < CK ? kd + kr * KP + c * 8 : vd + kr * VP + (c - CK) * 8;
      const long o = c < CK ? kofs[slot][kr] : vofs[slot][kr];
      if (o >= 0) fm_cp16((uint32_t)__cvta_generic_to_shared(dst), (c < CK ? A.kc + o + c * 8 : A.vc + o + (c - CK) * 8));
      else *(uint4*)dst = make_uint4(0u, 0u, 0u, 0u);
    }
  };

  locate(0, tile_at(0));
  if (n_tiles > 1) locate(1, tile_at(1));
  __syncthreads();
  load_tile(0, 0);
  fm_commit();

  // this thread's two rows (quad and quad + 8 of the warp's 16) and their query fragments
  const int ra = warp * 16 + quad, rb = ra + 8;
  const bool va = ra < rows, vb = rb < rows;
  const int pa = p0 + ra, pb = p0 + rb;
  int lo_a, keep_a, lo_b, keep_b;
  fm_lo_keep(A, pa, lo_a, keep_a);
  fm_lo_keep(A, pb, lo_b, keep_b);
  uint32_t qf[DK][4];
  {
    const __nv_bfloat16* qa = A.q + (size_t)(t0 + ra) * A.ldq + (size_t)h * D;
    const __nv_bfloat16* qb = A.q + (size_t)(t0 + rb) * A.ldq + (size_t)h * D;
#pragma unroll
    for (int ks = 0; ks < DK; ks++) {
      const int d = ks * 16 + qi * 2;
      qf[ks][0] = va ? *(const uint32_t*)(qa + d) : 0u;
      qf[ks][1] = vb ? *(const uint32_t*)(qb + d) : 0u;
      qf[ks][2] = va ? *(const uint32_t*)(qa + d + 8) : 0u;
      qf[ks][3] = vb ? *(const uint32_t*)(qb + d + 8) : 0u;
    }
  }
  float o[EN][4];
#pragma unroll
  for (int n = 0; n < EN; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

  // scores are kept in units of log 2 (scale * log2(e) folded into one factor): exp is then one exp2 an element
  const float sl2 = A.scale * 1.4426950408889634f;
  for (int it = 0; it < n_tiles; it++) {
    const int buf = it & 1, k0 = tile_at(it) * FM_KEYS;
    if (it + 1 < n_tiles) {
      load_tile(buf ^ 1, buf ^ 1);            // located an iteration ago; the barrier that ended it made that visible
      fm_commit();
      fm_wait<1>();
    } else {
      fm_wait<0>();
    }
    __syncthreads();
    if (it + 2 < n_tiles) locate(buf, tile_at(it + 2));     // this slot's copies are issued; visible after the next barrier
    const __nv_bfloat16* kt = Ks + buf * FM_KEYS * KP;
    const __nv_bfloat16* vt = Vs + buf * FM_KEYS * VP;
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    // lane l gives the row of matrix l / 8: keys (l / 16) * 8 + l % 8 of a pair of key tiles, columns ((l / 8) & 1) * 8
    const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(kt + ((lane >> 4) * 8 + (lane & 7)) * KP + ((lane >> 3) & 1) * 8);
#pragma unroll
    for (int ks = 0; ks < DK; ks++) {
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        uint32_t b[4];
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(k_addr + (uint32_t)((j * 8 * KP + ks * 16) * 2)));
        fm_mma(s[j], qf[ks], b[0], b[1]);
        fm_mma(s[j + 1], qf[ks], b[2], b[3]);
      }
    }
    // scale, mask, this tile's maximum
    float mx_a = -INFINITY, mx_b = -INFINITY;
    // a tile every key of which both rows see (the common case away from the diagonal and the mask's edge) needs no test
    const bool whole = va && vb && k0 + FM_KEYS - 1 <= pa && k0 >= lo_b;
    if (whole) {
#pragma unroll
      for (int j = 0; j < 8; j++) {
        s[j][0] *= sl2; s[j][1] *= sl2; s[j][2] *= sl2; s[j][3] *= sl2;
        mx_a = fmaxf(mx_a, fmaxf(s[j][0], s[j][1]));
        mx_b = fmaxf(mx_b, fmaxf(s[j][2], s[j][3]));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; j++) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
          const int key = k0 + j * 8 + qi * 2 + (c & 1);
          const bool top = c < 2;
          const int p = top ? pa : pb, lo = top ? lo_a : lo_b, keep = top ? keep_a : keep_b;
          const bool vis = (top ? va : vb) && key <= p && (key >= lo || key < keep);
          const float v = vis ? s[j][c] * sl2 : -INFINITY;
          s[j][c] = v;
          if (top) mx_a = fmaxf(mx_a, v); else mx_b = fmaxf(mx_b, v);
        }
      }
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
    const float al_a = mn_a == -INFINITY ? 1.f : exp2f(m_a - mn_a), al_b = mn_b == -INFINITY ? 1.f : exp2f(m_b - mn_b);
    m_a = mn_a;
    m_b = mn_b;
    float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      s[j][0] = mn_a == -INFINITY ? 0.f : exp2f(s[j][0] - mn_a);
      s[j][1] = mn_a == -INFINITY ? 0.f : exp2f(s[j][1] - mn_a);
      s[j][2] = mn_b == -INFINITY ? 0.f : exp2f(s[j][2] - mn_b);
      s[j][3] = mn_b == -INFINITY ? 0.f : exp2f(s[j][3] - mn_b);
      sum_a += s[j][0] + s[j][1];
      sum_b += s[j][2] + s[j][3];
    }
    l_a = fmaf(l_a, al_a, sum_a);
    l_b = fmaf(l_b, al_b, sum_b);
#pragma unroll
    for (int n = 0; n < EN; n++) { o[n][0] *= al_a; o[n][1] *= al_a; o[n][2] *= al_b; o[n][3] *= al_b; }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < 4; kk++) {
      uint32_t pf[4];
      pf[0] = fm_pack(s[2 * kk][0], s[2 * kk][1]);
      pf[1] = fm_pack(s[2 * kk][2], s[2 * kk][3]);
      pf[2] = fm_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pf[3] = fm_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
      // lane l gives the row of matrix l / 8: keys (l & 7) + ((l >> 3) & 1) * 8 of the 16, columns (l >> 4) * 8 of a pair of tiles
      const uint32_t vrow = (uint32_t)__cvta_generic_to_shared(vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VP + (lane >> 4) * 8);
#pragma unroll
      for (int n = 0; n + 1 < EN; n += 2) {
        uint32_t b[4];
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(vrow + n * 16));
        fm_mma(o[n], pf, b[0], b[1]);
        fm_mma(o[n + 1], pf, b[2], b[3]);
      }
    }
    __syncthreads();           // before the next iteration's copies overwrite the other buffer... and this one after it
  }
  // the rows' sums over the four threads of a quad, the sink, the gate
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  float f_a = 1.f, f_b = 1.f;
  if (A.sink) {
    const float sk = A.sink[h] * 1.4426950408889634f;       // the maxima are in units of log 2
    const float m2a = fmaxf(m_a, sk), m2b = fmaxf(m_b, sk);
    f_a = exp2f(m_a - m2a);
    l_a = fmaf(l_a, f_a, exp2f(sk - m2a));
    f_b = exp2f(m_b - m2b);
    l_b = fmaf(l_b, f_b, exp2f(sk - m2b));
  }
  f_a = l_a > 0.f ? f_a / l_a : 0.f;
  f_b = l_b > 0.f ? f_b / l_b : 0.f;
  const float* ga = A.gate ? A.gate + (size_t)(t0 + ra) * A.ld_gate + A.gate_off : nullptr;
  const float* gb = A.gate ? A.gate + (size_t)(t0 + rb) * A.ld_gate + A.gate_off : nullptr;
  if (A.gate_mode == 2) {
    if (va) f_a *= 1.f / (1.f + expf(-ga[h]));
    if (vb) f_b *= 1.f / (1.f + expf(-gb[h]));
  }
  TO* oa = (TO*)A.out + (size_t)(t0 + ra) * A.ldo + (size_t)h * E;
  TO* ob = (TO*)A.out + (size_t)(t0 + rb) * A.ldo + (size_t)h * E;
#pragma unroll
  for (int n = 0; n < EN; n++) {
    const int e = n * 8 + qi * 2;
    float x0 = o[n][0] * f_a, x1 = o[n][1] * f_a, y0 = o[n][2] * f_b, y1 = o[n][3] * f_b;
    if (A.gate_mode == 1) {
      if (va) { x0 *= 1.f / (1.f + expf(-ga[h * E + e])); x1 *= 1.f / (1.f + expf(-ga[h * E + e + 1])); }
      if (vb) { y0 *= 1.f / (1.f + expf(-gb[h * E + e])); y1 *= 1.f / (1.f + expf(-gb[h * E + e + 1])); }
    }
    if (va) { oa[e] = hb_from_float<TO>(x0); oa[e + 1] = hb_from_float<TO>(x1); }
    if (vb) { ob[e] = hb_from_float<TO>(y0); ob[e + 1] = hb_from_float<TO>(y1); }
  }
}

// the (D, E) pairs that are instantiated
#define FM_SIZES(X) X(4, 8) X(4, 6) X(8, 16) X(6, 8) X(12, 16) X(2, 4) X(4, 4) X(8, 8) X(3, 4)

HB_EXPORT int hb_attn_masked_flash_supported(int D, int E) {
#define FM_CHECK(DK, EN) if (D == 16 * DK && E == 8 * EN) return 1;
  FM_SIZES(FM_CHECK)
#undef FM_CHECK
  return 0;
}

HB_EXPORT int hb_attn_masked_flash(const void* q, long ldq, const void* kc, long k_page, long k_head, long k_row, const void* vc,
                                   long v_page, long v_head, long v_row, const int* bt, int bt_stride, const int* q_start,
                                   const int* q_len, const int* ctx_len, int req0, int n_requests, int max_q_len, int row_limit,
                                   const float* sink, const float* gate, long ld_gate, int gate_off, int gate_mode, void* out,
                                   int o_dt, long ldo, int H, int G, int D, int E, int page_size, int mask, int window,
                                   int keep_first, int chunk, float scale, cudaStream_t s) {
  if (n_requests <= 0 || max_q_len <= 0) return 0;
  if (G <= 0 || H % G) HB_FAIL("hb_attn_masked_flash: %d heads are not a multiple of %d kv heads", H, G);
  if (!hb_attn_masked_flash_supported(D, E)) HB_FAIL("hb_attn_masked_flash: keys of %d with values of %d are not a size it takes", D, E);
  if ((ldq | k_page | k_head | k_row | v_page | v_head | v_row) & 7 || (((uintptr_t)q | (uintptr_t)kc | (uintptr_t)vc) & 15))
    HB_FAIL("hb_attn_masked_flash: rows of q, keys and values must start on 16-byte boundaries");
  if (H > 65535 || n_requests > 65535) HB_FAIL("hb_attn_masked_flash: the grid is too large");
  FlashMaskedArgs A;
  A.q = (const __nv_bfloat16*)q; A.ldq = ldq; A.kc = (const __nv_bfloat16*)kc; A.k_page = k_page; A.k_head = k_head; A.k_row = k_row;
  A.vc = (const __nv_bfloat16*)vc; A.v_page = v_page; A.v_head = v_head; A.v_row = v_row; A.bt = bt; A.bt_stride = bt_stride;
  A.q_start = q_start; A.q_len = q_len; A.ctx_len = ctx_len; A.req0 = req0; A.row_limit = row_limit; A.sink = sink; A.gate = gate;
  A.ld_gate = ld_gate; A.gate_off = gate_off; A.gate_mode = gate ? gate_mode : 0; A.out = out; A.ldo = ldo; A.H = H; A.G = G;
  A.page_size = page_size; A.mask = mask; A.window = window; A.keep_first = keep_first; A.chunk = chunk; A.scale = scale;
  dim3 grid((max_q_len + FM_ROWS - 1) / FM_ROWS, H, n_requests);
#define FM_LAUNCH(DK, EN)                                                                                               \
  if (D == 16 * DK && E == 8 * EN) {                                                                                    \
    const size_t smem = (size_t)2 * FM_KEYS * ((16 * DK + 8) + (8 * EN + 8)) * sizeof(__nv_bfloat16);                   \
    if (o_dt == HB_BF16) {                                                                                              \
      auto kern = attn_masked_flash_kernel<DK, EN, __nv_bfloat16>;                                                      \
      if (smem + 4096 > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
      hb_launch(kern, grid, dim3(FM_THREADS), smem, s, A);                                                              \
    } else {                                                                                                            \
      auto kern = attn_masked_flash_kernel<DK, EN, float>;                                                              \
      if (smem + 4096 > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
      hb_launch(kern, grid, dim3(FM_THREADS), smem, s, A);                                                              \
    }                                                                                                                   \
  }
  FM_SIZES(FM_LAUNCH)
#undef FM_LAUNCH
  HB_CHECK_LAUNCH("hb_attn_masked_flash");
  return 0;
}
