// Attention of single rows (decoded tokens, short portions) over the paged cache on warp tensor-core instructions: the
// heads that share a kv head are the rows of the MMA tiles, so a key tile is read once for all of them. Mask, sink and
// gate as in attention_masked.cu (the same visibility rule; see there). bfloat16 queries, keys and values.
//
// One CTA of four warps per (kv head, row, tile of 16 MT heads of the group, key split). MT = 1 (up to 16 heads a tile)
// or 2 (up to 32); a warp owns one m-tile of 16 heads and one slice of the value columns (ES = 4 / MT slices), computes
// the scores of its heads against all 64 keys of a tile (warps of the same m-tile repeat that product: it is small
// beside the traffic), keeps the online softmax of its rows in registers, and accumulates its slice of O. Queries lie
// in shared memory (any D that is a multiple of 16), key and value tiles of 64 ABSOLUTE positions come by cp.async,
// double-buffered; the values may be the first E columns of the key rows (a latent that serves as both), in which case
// no value tile is loaded. A row's visible tiles are split HS_SPLIT_TILES a CTA (a matter of its position alone). A
// row that one CTA walks is finished by it (sink, gate, one rounding); the partial results of a row that several walk
// are joined, in the splits' order, by a second kernel over the whole machine.
#include "common.cuh"

#define HK 64
constexpr int HS_THREADS = 128, HS_SPLIT_TILES = 4;

struct HeadsArgs {
  const __nv_bfloat16* q; long ldq;
  const __nv_bfloat16* kc; long k_page, k_head, k_row;
  const __nv_bfloat16* vc; long v_page, v_head, v_row;
  int alias;                            // values are the first E columns of the key rows
  const int* bt; int bt_stride;
  const int* row_req; const int* pos;
  const float* sink;
  const float* gate; long ld_gate; int gate_off; int gate_mode;
  void* out; long ldo;
  int H, G, D, E, MT, page_size, mask, window, keep_first, chunk;
  float scale;
  const int* q_len; int row_limit;
  float* part;                          // [T][G][ZT][splits][16 MT][E + 4]
  int splits;
};

__device__ __forceinline__ void hs_cp16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void hs_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t hs_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}
__host__ __device__ __forceinline__ int hs_tile_count(int p, int lo, int keep) {
  const int last = p / HK, first_win = lo / HK, last_keep = keep > 0 ? (keep - 1) / HK : -1;
  if (first_win <= last_keep + 1) return last + 1;
  return (last_keep + 1) + (last - first_win + 1);
}
__device__ __forceinline__ int hs_tile_at(int i, int lo, int keep) {
  const int first_win = lo / HK, last_keep = keep > 0 ? (keep - 1) / HK : -1;
  if (first_win <= last_keep + 1 || i <= last_keep) return i;
  return first_win + (i - (last_keep + 1));
}

template <int ENW, typename TO>
__global__ void __launch_bounds__(HS_THREADS) attn_masked_heads_kernel(HeadsArgs A) {
  extern __shared__ __align__(16) uint8_t hs_smem[];
  hb_pdl_launch();
  hb_pdl_wait();
  const int g = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, quad = lane >> 2, qi = lane & 3;
  const int ZT = gridDim.z / A.splits, z = blockIdx.z / A.splits, split = blockIdx.z % A.splits;
  if (A.q_len && A.q_len[A.row_req[t]] >= A.row_limit) return;
  const int D = A.D, E = A.E, MT = A.MT, MR = 16 * MT, HG = A.H / A.G, ps = A.page_size;
  const int KP = D + 8, VP = A.alias ? KP : E + 8;
  const int h0 = z * MR, nh = min(MR, HG - h0);
  __nv_bfloat16* Qs = (__nv_bfloat16*)hs_smem;              // [MR][KP]
  __nv_bfloat16* Ks = Qs + MR * KP;                          // [2][HK][KP]
  __nv_bfloat16* Vs = A.alias ? Ks : Ks + 2 * HK * KP;       // [2][HK][VP]
  const int p = A.pos[t];
  int lo = 0, keep = 0;
  if (A.mask == 1 && A.window > 0) { lo = max(0, p - A.window + 1); keep = min(A.keep_first, p + 1); }
  else if (A.mask == 2 && A.chunk > 0) lo = (p / A.chunk) * A.chunk;
  const int n_tiles = hs_tile_count(p, lo, keep);
  const int n_splits_row = (n_tiles + HS_SPLIT_TILES - 1) / HS_SPLIT_TILES;       // a matter of the row's position alone
  if (split >= n_splits_row) return;
  const int i0 = split * HS_SPLIT_TILES, i1 = min(n_tiles, i0 + HS_SPLIT_TILES);
  const int* table = A.bt + (size_t)A.row_req[t] * A.bt_stride;

  // where a tile's 64 keys lie is looked up once a tile, by one thread a key, a tile before the copies that use it
  __shared__ long kofs[2][HK], vofs[2][HK];
  auto locate = [&](int slot, int tile) {
    if (tid < HK) {
      const int kp = tile * HK + tid;
      const bool vis = kp <= p && (kp >= lo || kp < keep);
      const int page = vis ? table[kp / ps] : -1;
      const int off = kp % ps;
      kofs[slot][tid] = page >= 0 ? (long)page * A.k_page + (long)g * A.k_head + (long)off * A.k_row : -1;
      vofs[slot][tid] = page >= 0 ? (long)page * A.v_page + (long)g * A.v_head + (long)off * A.v_row : -1;
    }
  };
  auto load_tile = [&](int buf, int slot) {
    const int CK = D / 8, CV = A.alias ? 0 : E / 8;
    __nv_bfloat16* kd = Ks + buf * HK * KP;
    __nv_bfloat16* vd = Vs + buf * HK * VP;
    for (int i = tid; i < HK * (CK + CV); i += HS_THREADS) {
      const int kr = i / (CK + CV), c = i - kr * (CK + CV);
      __nv_bfloat16* dst = c < CK ? kd + kr * KP + c * 8 : vd + kr * VP + (c - CK) * 8;
      const long o = c < CK ? kofs[slot][kr] : vofs[slot][kr];
      if (o >= 0) hs_cp16((uint32_t)__cvta_generic_to_shared(dst), (c < CK ? A.kc + o + c * 8 : A.vc + o + (c - CK) * 8));
      else *(uint4*)dst = make_uint4(0u, 0u, 0u, 0u);
    }
  };
  locate(0, hs_tile_at(i0, lo, keep));
  if (i0 + 1 < i1) locate(1, hs_tile_at(i0 + 1, lo, keep));
  __syncthreads();
  load_tile(0, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");
  // the queries of the tile's heads (rows beyond the group's heads are zero)
  {
    const __nv_bfloat16* qrow = A.q + (size_t)t * A.ldq + ((size_t)g * HG + h0) * D;
    const int CQ = D / 8;
    for (int i = tid; i < MR * CQ; i += HS_THREADS) {
      const int r = i / CQ, c = i - r * CQ;
      *(uint4*)(Qs + r * KP + c * 8) = r < nh ? *(const uint4*)(qrow + (size_t)r * D + c * 8) : make_uint4(0u, 0u, 0u, 0u);
    }
  }
  const int mt = warp % MT, es = warp / MT, e_base = es * ENW * 8;
  float o[ENW][4];
#pragma unroll
  for (int n = 0; n < ENW; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(Qs + (mt * 16 + (lane & 15)) * KP + (lane >> 4) * 8);

  // scores are kept in units of log 2 (scale * log2(e) folded into one factor): exp is then one exp2 an element
  const float sl2 = A.scale * 1.4426950408889634f;
  for (int it = i0; it < i1; it++) {
    const int buf = (it - i0) & 1, k0 = hs_tile_at(it, lo, keep) * HK;
    if (it + 1 < i1) {
      load_tile(buf ^ 1, buf ^ 1);            // located an iteration ago (or before the loop)
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    if (it + 2 < i1) locate(buf, hs_tile_at(it + 2, lo, keep));
    const __nv_bfloat16* kt = Ks + buf * HK * KP;
    const __nv_bfloat16* vt = Vs + buf * HK * VP;
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    // lane l gives the row of matrix l / 8: keys (l / 16) * 8 + l % 8 of a pair of key tiles, columns ((l / 8) & 1) * 8
    const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(kt + ((lane >> 4) * 8 + (lane & 7)) * KP + ((lane >> 3) & 1) * 8);
    for (int ks = 0; ks < D / 16; ks++) {
      uint32_t a[4];
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                   : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(q_addr + ks * 32));
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        uint32_t b[4];
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(k_addr + (uint32_t)(j * 8 * KP * 2 + ks * 32)));
        hs_mma(s[j], a, b[0], b[1]);
        hs_mma(s[j + 1], a, b[2], b[3]);
      }
    }
    float mx = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; j++) {
#pragma unroll
      for (int c = 0; c < 4; c++) {
        const int key = k0 + j * 8 + qi * 2 + (c & 1);
        const bool vis = key <= p && (key >= lo || key < keep);
        const float v = vis ? s[j][c] * sl2 : -INFINITY;
        s[j][c] = v;
        if (c < 2) mx = fmaxf(mx, v); else mx_b = fmaxf(mx_b, v);
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx), mn_b = fmaxf(m_b, mx_b);
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
    for (int n = 0; n < ENW; n++) { o[n][0] *= al_a; o[n][1] *= al_a; o[n][2] *= al_b; o[n][3] *= al_b; }
    // lane l gives the row of matrix l / 8: keys (l & 7) + ((l >> 3) & 1) * 8 of a group of 16, columns (l >> 4) * 8 of a pair
    const uint32_t v_addr = (uint32_t)__cvta_generic_to_shared(vt + ((lane & 7) + ((lane >> 3) & 1) * 8) * VP + e_base + (lane >> 4) * 8);
#pragma unroll
    for (int kk = 0; kk < 4; kk++) {
      uint32_t pf[4];
      pf[0] = hs_pack(s[2 * kk][0], s[2 * kk][1]);
      pf[1] = hs_pack(s[2 * kk][2], s[2 * kk][3]);
      pf[2] = hs_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pf[3] = hs_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int n = 0; n < ENW; n += 2) {
        uint32_t b[4];
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(v_addr + (uint32_t)((kk * 16 * VP + n * 8) * 2)));
        hs_mma(o[n], pf, b[0], b[1]);
        hs_mma(o[n + 1], pf, b[2], b[3]);
      }
    }
    __syncthreads();
  }
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  const int ra = mt * 16 + quad, rb = ra + 8;        // this thread's two heads of the tile
  // the accumulators, maxima and sums go through memory: shared (one split) or the workspace (several)
  float* stage;
  const size_t slot = ((size_t)t * A.G + g) * ZT + z;
  const int RS = E + 4;                 // a row's sums, then its maximum and weight sum; rows stay 16-byte aligned
  if (n_splits_row > 1) stage = A.part + (slot * A.splits + split) * (size_t)MR * RS;
  else stage = (float*)hs_smem;                       // the tiles are done with
  __syncthreads();
#pragma unroll
  for (int n = 0; n < ENW; n++) {
    const int e = e_base + n * 8 + qi * 2;
    stage[ra * RS + e] = o[n][0]; stage[ra * RS + e + 1] = o[n][1];
    stage[rb * RS + e] = o[n][2]; stage[rb * RS + e + 1] = o[n][3];
  }
  if (es == 0 && qi == 0) {
    stage[ra * RS + E] = m_a; stage[ra * RS + E + 1] = l_a;
    stage[rb * RS + E] = m_b; stage[rb * RS + E + 1] = l_b;
  }
  if (n_splits_row > 1) return;            // the merge kernel joins the splits of such a row
  const float* all = stage;
  const int n_parts = 1;
  __syncthreads();
  const size_t pstride = (size_t)MR * RS;
  // every head's factor for each split (exp of the split's maximum against the row's, over the weight sum with the sink,
  // times the head's gate) first, into shared memory behind the staged sums; then every (head, 4 columns) is one
  // thread's sum over the splits, all loads independent of one another
  float* wsp = (float*)hs_smem + (size_t)MR * RS;            // [nh][n_parts], n_parts <= 64 here
  const bool use_table = n_parts <= 64;
  if (use_table) {
    for (int r = tid; r < nh; r += HS_THREADS) {
      const size_t head = (size_t)g * HG + h0 + r;
      float m = -INFINITY;
      for (int sp = 0; sp < n_parts; sp++) m = fmaxf(m, all[sp * pstride + r * RS + E]);
      float l = 0.f;
      for (int sp = 0; sp < n_parts; sp++) l = fmaf(all[sp * pstride + r * RS + E + 1], exp2f(all[sp * pstride + r * RS + E] - m), l);
      float f = 1.f;
      if (A.sink) {
        const float sk = A.sink[head] * 1.4426950408889634f, m2 = fmaxf(m, sk);     // the maxima are in units of log 2
        f = exp2f(m - m2);
        l = fmaf(l, f, exp2f(sk - m2));
      }
      f = l > 0.f ? f / l : 0.f;
      if (A.gate_mode == 2) f *= 1.f / (1.f + expf(-A.gate[(size_t)t * A.ld_gate + A.gate_off + head]));
      for (int sp = 0; sp < n_parts; sp++) wsp[r * n_parts + sp] = exp2f(all[sp * pstride + r * RS + E] - m) * f;
    }
    __syncthreads();
    const int C4 = E / 4;
    for (int i = tid; i < nh * C4; i += HS_THREADS) {
      const int r = i / C4, e = (i - r * C4) * 4;
      const size_t head = (size_t)g * HG + h0 + r;
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
      for (int sp = 0; sp < n_parts; sp++) {
        const float4 v = *(const float4*)(all + sp * pstride + r * RS + e);
        const float w = wsp[r * n_parts + sp];
        a.x = fmaf(v.x, w, a.x); a.y = fmaf(v.y, w, a.y); a.z = fmaf(v.z, w, a.z); a.w = fmaf(v.w, w, a.w);
      }
      if (A.gate_mode == 1) {
        const float* gp = A.gate + (size_t)t * A.ld_gate + A.gate_off + head * E + e;
        a.x *= 1.f / (1.f + expf(-gp[0])); a.y *= 1.f / (1.f + expf(-gp[1]));
        a.z *= 1.f / (1.f + expf(-gp[2])); a.w *= 1.f / (1.f + expf(-gp[3]));
      }
      TO* op = (TO*)A.out + (size_t)t * A.ldo + head * E + e;
      op[0] = hb_from_float<TO>(a.x); op[1] = hb_from_float<TO>(a.y); op[2] = hb_from_float<TO>(a.z); op[3] = hb_from_float<TO>(a.w);
    }
    return;
  }
  for (int r = warp; r < nh; r += HS_THREADS / 32) {
    const size_t head = (size_t)g * HG + h0 + r;
    float m = -INFINITY;
    for (int sp = 0; sp < n_parts; sp++) m = fmaxf(m, all[sp * pstride + r * RS + E]);
    float l = 0.f;
    for (int sp = 0; sp < n_parts; sp++) l = fmaf(all[sp * pstride + r * RS + E + 1], exp2f(all[sp * pstride + r * RS + E] - m), l);
    float f = 1.f;
    if (A.sink) {
      const float sk = A.sink[head] * 1.4426950408889634f, m2 = fmaxf(m, sk);
      f = exp2f(m - m2);
      l = fmaf(l, f, exp2f(sk - m2));
    }
    f = l > 0.f ? f / l : 0.f;
    float gh = 1.f;
    if (A.gate_mode == 2) gh = 1.f / (1.f + expf(-A.gate[(size_t)t * A.ld_gate + A.gate_off + head]));
    for (int e = lane; e < E; e += 32) {
      float a = 0.f;
      for (int sp = 0; sp < n_parts; sp++) a = fmaf(all[sp * pstride + r * RS + e], exp2f(all[sp * pstride + r * RS + E] - m), a);
      a *= f;
      if (A.gate_mode == 1) a *= 1.f / (1.f + expf(-A.gate[(size_t)t * A.ld_gate + A.gate_off + head * E + e]));
      else if (A.gate_mode == 2) a *= gh;
      ((TO*)A.out)[(size_t)t * A.ldo + head * E + e] = hb_from_float<TO>(a);
    }
  }
}

// Joins the key splits of rows that were walked by several CTAs: one thread a (head, 4 value columns). It finds the row's
// maximum and weight sum over the splits (a few cached loads), adds the sink, and sums the splits' columns times
// exp2(split maximum - row maximum) in the splits' order, all loads independent of one another; gate and one rounding
// on the way out. The whole machine takes part: the partial sums of a latent layer's row are as large as a third of
// the keys it read, too much for one CTA to pull through its own loads.
template <typename TO>
__global__ void __launch_bounds__(HS_THREADS) attn_masked_heads_merge_kernel(HeadsArgs A) {
  hb_pdl_launch();
  hb_pdl_wait();
  const int t = blockIdx.z, ZT = gridDim.y / A.G, g = blockIdx.y / ZT, z = blockIdx.y % ZT;
  if (A.q_len && A.q_len[A.row_req[t]] >= A.row_limit) return;
  const int E = A.E, MR = 16 * A.MT, HG = A.H / A.G, RS = E + 4, C4 = E / 4;
  const int h0 = z * MR, nh = min(MR, HG - h0);
  const int p = A.pos[t];
  int lo = 0, keep = 0;
  if (A.mask == 1 && A.window > 0) { lo = max(0, p - A.window + 1); keep = min(A.keep_first, p + 1); }
  else if (A.mask == 2 && A.chunk > 0) lo = (p / A.chunk) * A.chunk;
  const int n_parts = (hs_tile_count(p, lo, keep) + HS_SPLIT_TILES - 1) / HS_SPLIT_TILES;
  if (n_parts <= 1) return;                                   // finished by the CTA that walked it
  const int i = blockIdx.x * HS_THREADS + threadIdx.x;
  if (i >= nh * C4) return;
  const int r = i / C4, e = (i - r * C4) * 4;
  const size_t slot = ((size_t)t * A.G + g) * ZT + z, pstride = (size_t)MR * RS;
  const float* all = A.part + slot * A.splits * pstride + (size_t)r * RS;
  const size_t head = (size_t)g * HG + h0 + r;
  float m = -INFINITY;
  for (int sp = 0; sp < n_parts; sp++) m = fmaxf(m, all[sp * pstride + E]);
  float l = 0.f;
  for (int sp = 0; sp < n_parts; sp++) l = fmaf(all[sp * pstride + E + 1], exp2f(all[sp * pstride + E] - m), l);
  float f = 1.f;
  if (A.sink) {
    const float sk = A.sink[head] * 1.4426950408889634f, m2 = fmaxf(m, sk);     // the maxima are in units of log 2
    f = exp2f(m - m2);
    l = fmaf(l, f, exp2f(sk - m2));
  }
  f = l > 0.f ? f / l : 0.f;
  if (A.gate_mode == 2) f *= 1.f / (1.f + expf(-A.gate[(size_t)t * A.ld_gate + A.gate_off + head]));
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
  for (int sp = 0; sp < n_parts; sp++) {
    const float4 v = *(const float4*)(all + sp * pstride + e);
    const float w = exp2f(all[sp * pstride + E] - m);
    a.x = fmaf(v.x, w, a.x); a.y = fmaf(v.y, w, a.y); a.z = fmaf(v.z, w, a.z); a.w = fmaf(v.w, w, a.w);
  }
  a.x *= f; a.y *= f; a.z *= f; a.w *= f;
  if (A.gate_mode == 1) {
    const float* gp = A.gate + (size_t)t * A.ld_gate + A.gate_off + head * E + e;
    a.x *= 1.f / (1.f + expf(-gp[0])); a.y *= 1.f / (1.f + expf(-gp[1]));
    a.z *= 1.f / (1.f + expf(-gp[2])); a.w *= 1.f / (1.f + expf(-gp[3]));
  }
  TO* op = (TO*)A.out + (size_t)t * A.ldo + head * E + e;
  op[0] = hb_from_float<TO>(a.x); op[1] = hb_from_float<TO>(a.y); op[2] = hb_from_float<TO>(a.z); op[3] = hb_from_float<TO>(a.w);
}

static int hs_mt(int HG) { return HG > 16 ? 2 : 1; }
static size_t hs_smem_bytes(int MT, int D, int E, int alias) {
  size_t tiles = (size_t)(16 * MT) * (D + 8) * 2 + (size_t)2 * HK * (D + 8) * 2 + (alias ? 0 : (size_t)2 * HK * (E + 8) * 2);
  size_t stage = (size_t)(16 * MT) * (E + 4) * 4 + (size_t)(16 * MT) * 64 * 4;   // one split's sums, and the splits' weights
  return tiles > stage ? tiles : stage;
}
static int hs_splits(int mask, int window, int keep_first, int chunk, int max_pos) {
  int worst = max_pos / HK + 1;
  if (mask == 1 && window > 0) {
    const int w = (window - 1 + HK - 1) / HK + 1 + (keep_first > 0 ? (keep_first - 1) / HK + 1 : 0);
    if (w < worst) worst = w;
  } else if (mask == 2 && chunk > 0) {
    const int w = (chunk - 1 + HK - 1) / HK + 1;
    if (w < worst) worst = w;
  }
  return (worst + HS_SPLIT_TILES - 1) / HS_SPLIT_TILES;
}

// value columns a warp owns, in tiles of 8, for these sizes; 0: not a size the kernel takes
static int hs_enw(int H, int G, int D, int E, int alias) {
  if (G <= 0 || H % G || D % 16 || E % 8 || D > 1024) return 0;
  const int MT = hs_mt(H / G), ES = 4 / MT;
  if (E % (8 * ES)) return 0;
  const int enw = E / 8 / ES;
  if (enw != 2 && enw != 4 && enw != 8 && enw != 16 && enw != 32) return 0;
  if (alias && E > D) return 0;
  if (hs_smem_bytes(MT, D, E, alias) > 200 * 1024) return 0;
  return enw;
}

HB_EXPORT int hb_attn_masked_heads_supported(int H, int G, int D, int E, int alias) { return hs_enw(H, G, D, E, alias) ? 1 : 0; }

HB_EXPORT long hb_attn_masked_heads_workspace(int T, int H, int G, int E, int mask, int window, int keep_first, int chunk, int max_pos) {
  const int HG = H / G, MT = hs_mt(HG), ZT = (HG + 16 * MT - 1) / (16 * MT);
  const int splits = hs_splits(mask, window, keep_first, chunk, max_pos);
  if (splits <= 1) return 0;
  return (long)T * G * ZT * splits * 16 * MT * (E + 4);
}
HB_EXPORT int hb_attn_masked_heads(const void* q, long ldq, const void* kc, long k_page, long k_head, long k_row, const void* vc,
                                   long v_page, long v_head, long v_row, int alias, const int* bt, int bt_stride,
                                   const int* row_req, const int* pos, const float* sink, const float* gate, long ld_gate,
                                   int gate_off, int gate_mode, void* out, int o_dt, long ldo, int T, int H, int G, int D, int E,
                                   int page_size, int mask, int window, int keep_first, int chunk, float scale, const int* q_len,
                                   int row_limit, float* part, long n_part, int max_pos, cudaStream_t s) {
  if (T <= 0) return 0;
  const int enw = hs_enw(H, G, D, E, alias);
  if (!enw) HB_FAIL("hb_attn_masked_heads: %d heads over %d kv heads with keys of %d and values of %d are not sizes it takes", H, G, D, E);
  if (T > 65535) HB_FAIL("hb_attn_masked_heads: %d rows are beyond the grid limit", T);
  if ((ldq | k_page | k_head | k_row | v_page | v_head | v_row) & 7 || (((uintptr_t)q | (uintptr_t)kc | (uintptr_t)vc) & 15))
    HB_FAIL("hb_attn_masked_heads: rows of q, keys and values must start on 16-byte boundaries");
  HeadsArgs A;
  A.q = (const __nv_bfloat16*)q; A.ldq = ldq; A.kc = (const __nv_bfloat16*)kc; A.k_page = k_page; A.k_head = k_head; A.k_row = k_row;
  A.vc = (const __nv_bfloat16*)vc; A.v_page = v_page; A.v_head = v_head; A.v_row = v_row; A.alias = alias; A.bt = bt;
  A.bt_stride = bt_stride; A.row_req = row_req; A.pos = pos; A.sink = sink; A.gate = gate; A.ld_gate = ld_gate; A.gate_off = gate_off;
  A.gate_mode = gate ? gate_mode : 0; A.out = out; A.ldo = ldo; A.H = H; A.G = G; A.D = D; A.E = E; A.page_size = page_size;
  A.mask = mask; A.window = window; A.keep_first = keep_first; A.chunk = chunk; A.scale = scale; A.q_len = q_len;
  A.row_limit = row_limit; A.part = part;
  const int HG = H / G;
  A.MT = hs_mt(HG);
  const int ZT = (HG + 16 * A.MT - 1) / (16 * A.MT);
  A.splits = hs_splits(mask, window, keep_first, chunk, max_pos);
  if (A.splits < 1) A.splits = 1;
  if (A.splits > 1 && (!part || n_part < (long)T * G * ZT * A.splits * 16 * A.MT * (E + 4)))
    HB_FAIL("hb_attn_masked_heads: rows of up to %d key tiles need a workspace", A.splits * HS_SPLIT_TILES);
  if ((long)ZT * A.splits > 65535) HB_FAIL("hb_attn_masked_heads: the grid is too large");
  const size_t smem = hs_smem_bytes(A.MT, D, E, alias);
  dim3 grid(G, T, ZT * A.splits);
#define HS_LAUNCH(ENW)                                                                                              \
  if (enw == ENW) {                                                                                                 \
    if (o_dt == HB_BF16) {                                                                                          \
      auto kern = attn_masked_heads_kernel<ENW, __nv_bfloat16>;                                                     \
      if (smem + 4096 > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
      hb_launch(kern, grid, dim3(HS_THREADS), smem, s, A);                                                          \
    } else {                                                                                                        \
      auto kern = attn_masked_heads_kernel<ENW, float>;                                                             \
      if (smem + 4096 > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
      hb_launch(kern, grid, dim3(HS_THREADS), smem, s, A);                                                          \
    }                                                                                                               \
  }
  HS_LAUNCH(2) HS_LAUNCH(4) HS_LAUNCH(8) HS_LAUNCH(16) HS_LAUNCH(32)
#undef HS_LAUNCH
  HB_CHECK_LAUNCH("hb_attn_masked_heads");
  if (A.splits > 1) {
    dim3 mgrid((16 * A.MT * (E / 4) + HS_THREADS - 1) / HS_THREADS, G * ZT, T);
    if (o_dt == HB_BF16) hb_launch(attn_masked_heads_merge_kernel<__nv_bfloat16>, mgrid, dim3(HS_THREADS), 0, s, A);
    else hb_launch(attn_masked_heads_merge_kernel<float>, mgrid, dim3(HS_THREADS), 0, s, A);
    HB_CHECK_LAUNCH("hb_attn_masked_heads (merge)");
  }
  return 0;
}
