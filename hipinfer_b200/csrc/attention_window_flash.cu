// Flash attention for prompt portions with a window that keeps the first tokens and TWO score maps per head
// (differential attention), over the paged bf16 cache: the tensor-core counterpart of attention_window.cu for
// requests that bring at least `min_rows` rows.
//
// One CTA = 64 consecutive query rows of one request and one query head (4 warps x 16 rows), both maps. It walks the
// keys that any of its rows can see in tiles of 64 ABSOLUTE positions: the tiles of the kept first tokens, then the
// tiles from the window's start of its first row to its last row's position. A tile's keys [64][2 D] (map 0 | map 1)
// and values [64][E] are gathered page by page with cp.async into swizzled shared memory (double-buffered); per map
// S = Q K^T and O += P V run on warp MMAs (m16n8k16, bf16 in, fp32 out) with an online softmax of its own (exp2 domain,
// fp32; P rounded to bf16 before P V). At the end, per row: o = O_0 / l_0 - lambda O_1 / l_1, divided by its root mean
// square over the E values, times `post`, times sigmoid(gate), rounded once. A key that no row of the CTA can see is
// never read (its page may have been given back). Tiles are cut at absolute positions and a row's running maximum
// and sum are its own, so a row's result does not depend on how the prompt was cut or on the batch.
#include "tc_common.cuh"

constexpr int WF_BQ = 64, WF_BKV = 64, WF_THREADS = 128;

__device__ __forceinline__ uint32_t wf_swz(int row, int chunk, int row_bytes) {
  return (uint32_t)(row * row_bytes + ((chunk ^ (row & 7)) << 4));
}

struct WinFlashArgs {
  const __nv_bfloat16* q;    // [T][H][2 D]
  const __nv_bfloat16* kc;   // [page][G][page_size][2 D]
  const __nv_bfloat16* vc;   // [page][G][page_size][E]
  const int* bt;
  int bt_stride;
  const int* q_start;
  const int* q_len;
  const int* ctx_len;
  const float* gate;         // [T][ld_gate] at column gate_off, or null
  long ld_gate;
  int gate_off;
  __nv_bfloat16* out;        // [T][H][E]
  int H, G, page_size, window, keep_first;
  float scale_log2, lambda, post, eps;
  int min_rows;
};

// Rows [k_base, k_base + 64) of a plane whose rows are W elements wide into a swizzled [64][W] tile; a row that no
// query of the CTA sees is zeroed instead.
template <int W>
__device__ __forceinline__ void wf_load_tile(uint32_t tile, const __nv_bfloat16* __restrict__ cache, const int* __restrict__ table,
                                             int G, int h, int page_size, int k_base, int lo, int keep, int p_last, int tid) {
  constexpr int CH = W / 8;
  for (int i = tid; i < WF_BKV * CH; i += WF_THREADS) {
    const int r = i / CH, c = i - r * CH, kp = k_base + r;
    const uint32_t dst = tile + wf_swz(r, c, W * 2);
    if (kp <= p_last && (kp >= lo || kp < keep)) {
      const size_t page = table[kp / page_size];
      hb_cp_async16(dst, cache + ((page * G + h) * page_size + kp % page_size) * W + c * 8);
    } else {
      asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
    }
  }
}

template <int D, int E>
__global__ void __launch_bounds__(WF_THREADS) attn_window_flash_kernel(WinFlashArgs A) {
  constexpr int QW = 2 * D, KS = D / 16, NT_O = E / 8, KTILE = WF_BKV * QW * 2, VTILE = WF_BKV * E * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  hb_pdl_launch();
  hb_pdl_wait();
  const int req = blockIdx.z, hq = blockIdx.x, qt = gridDim.y - 1 - blockIdx.y;     // heaviest query tiles first
  const int n_rows = A.q_len[req];
  if (n_rows < A.min_rows || qt * WF_BQ >= n_rows) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int H = A.H, G = A.G, h = hq / (H / G), window = A.window;
  const int row0 = A.q_start[req] + qt * WF_BQ, rows_here = min(WF_BQ, n_rows - qt * WF_BQ);
  const int p_first = A.ctx_len[req] + qt * WF_BQ, p_last = p_first + rows_here - 1;
  const int* table = A.bt + (size_t)req * A.bt_stride;
  const uint32_t sQ = hb_smem_u32(smem), sK = sQ + WF_BQ * QW * 2, sV = sK + 2 * KTILE;

  for (int i = tid; i < WF_BQ * (QW / 8); i += WF_THREADS) {
    const int r = i / (QW / 8), c = i - r * (QW / 8);
    const uint32_t dst = sQ + wf_swz(r, c, QW * 2);
    if (r < rows_here) hb_cp_async16(dst, A.q + ((size_t)(row0 + r) * H + hq) * QW + c * 8);
    else asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
  }
  const int lo = window > 0 ? max(0, p_first - window + 1) : 0;
  const int keep = window > 0 ? min(A.keep_first, p_last + 1) : 0;
  const int kt_lo = lo / WF_BKV, kt_hi = p_last / WF_BKV;
  const int keep_hi = keep > 0 ? (keep - 1) / WF_BKV : -1;       // the last tile of kept tokens
  int kt = keep_hi >= 0 ? 0 : kt_lo;
  wf_load_tile<QW>(sK, A.kc, table, G, h, A.page_size, kt * WF_BKV, lo, keep, p_last, tid);
  wf_load_tile<E>(sV, A.vc, table, G, h, A.page_size, kt * WF_BKV, lo, keep, p_last, tid);
  hb_cp_async_commit();
  hb_cp_async_wait<0>();
  __syncthreads();

  float o[2][NT_O][4];
#pragma unroll
  for (int m = 0; m < 2; m++)
#pragma unroll
    for (int i = 0; i < NT_O; i++) o[m][i][0] = o[m][i][1] = o[m][i][2] = o[m][i][3] = 0.f;
  float mx[2][2] = {{-INFINITY, -INFINITY}, {-INFINITY, -INFINITY}}, ls[2][2] = {{0.f, 0.f}, {0.f, 0.f}};   // [map][row a, b]
  const int r_a = warp * 16 + g, r_b = r_a + 8;
  const int qp_a = p_first + min(r_a, rows_here - 1), qp_b = p_first + min(r_b, rows_here - 1);
  const int mi = lane >> 3, lr = lane & 7;

  for (int it = 0; kt <= kt_hi; it++) {
    const int buf = it & 1;
    const int next = (kt == keep_hi && kt + 1 < kt_lo) ? kt_lo : kt + 1;
    if (next <= kt_hi) {
      wf_load_tile<QW>(sK + (buf ^ 1) * KTILE, A.kc, table, G, h, A.page_size, next * WF_BKV, lo, keep, p_last, tid);
      wf_load_tile<E>(sV + (buf ^ 1) * VTILE, A.vc, table, G, h, A.page_size, next * WF_BKV, lo, keep, p_last, tid);
    }
    hb_cp_async_commit();
    const uint32_t tK = sK + buf * KTILE, tV = sV + buf * VTILE;
    const int k_base = kt * WF_BKV;
    const bool all_seen = k_base + WF_BKV - 1 <= p_first &&
                          (window <= 0 || k_base >= p_last - window + 1 || k_base + WF_BKV - 1 < keep);
#pragma unroll
    for (int m = 0; m < 2; m++) {
      float s[8][4];
#pragma unroll
      for (int i = 0; i < 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < KS; kk++) {
        uint32_t a[4];
        hb_ldmatrix_x4(a, sQ + wf_swz(warp * 16 + (mi & 1) * 8 + lr, m * (D / 8) + kk * 2 + (mi >> 1), QW * 2));
#pragma unroll
        for (int np = 0; np < 4; np++) {
          uint32_t b[4];
          hb_ldmatrix_x4(b, tK + wf_swz(np * 16 + (mi >> 1) * 8 + lr, m * (D / 8) + kk * 2 + (mi & 1), QW * 2));
          hb_mma_16816(s[2 * np], a, b);
          hb_mma_16816(s[2 * np + 1], a, b + 2);
        }
      }
      float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
      for (int i = 0; i < 8; i++) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
          if (!all_seen) {
            const int kp = k_base + i * 8 + 2 * t + e;
            const bool kept = kp < keep;
            if (!(kp <= qp_a && (window <= 0 || kp > qp_a - window || kept))) s[i][e] = -INFINITY;
            if (!(kp <= qp_b && (window <= 0 || kp > qp_b - window || kept))) s[i][2 + e] = -INFINITY;
          }
          mx_a = fmaxf(mx_a, s[i][e]);
          mx_b = fmaxf(mx_b, s[i][2 + e]);
        }
      }
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
      const float mn_a = fmaxf(mx[m][0], mx_a * A.scale_log2), mn_b = fmaxf(mx[m][1], mx_b * A.scale_log2);
      const float sub_a = mn_a == -INFINITY ? 0.f : mn_a, sub_b = mn_b == -INFINITY ? 0.f : mn_b;
      const float corr_a = hb_exp2(mx[m][0] - sub_a), corr_b = hb_exp2(mx[m][1] - sub_b);
      mx[m][0] = mn_a; mx[m][1] = mn_b;
      float sum_a = 0.f, sum_b = 0.f;
      uint32_t pf[4][4];
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const float p0 = hb_exp2(s[i][0] * A.scale_log2 - sub_a), p1 = hb_exp2(s[i][1] * A.scale_log2 - sub_a);
        const float p2 = hb_exp2(s[i][2] * A.scale_log2 - sub_b), p3 = hb_exp2(s[i][3] * A.scale_log2 - sub_b);
        sum_a += p0 + p1;
        sum_b += p2 + p3;
        pf[i >> 1][(i & 1) * 2] = hb_pack_bf16(p0, p1);
        pf[i >> 1][(i & 1) * 2 + 1] = hb_pack_bf16(p2, p3);
      }
      ls[m][0] = ls[m][0] * corr_a + sum_a;
      ls[m][1] = ls[m][1] * corr_b + sum_b;
#pragma unroll
      for (int i = 0; i < NT_O; i++) { o[m][i][0] *= corr_a; o[m][i][1] *= corr_a; o[m][i][2] *= corr_b; o[m][i][3] *= corr_b; }
#pragma unroll
      for (int j2 = 0; j2 < 4; j2++) {
#pragma unroll
        for (int cp = 0; cp < NT_O / 2; cp++) {
          uint32_t b[4];
          hb_ldmatrix_x4_trans(b, tV + wf_swz(j2 * 16 + (mi & 1) * 8 + lr, cp * 2 + (mi >> 1), E * 2));
          hb_mma_16816(o[m][2 * cp], pf[j2], b);
          hb_mma_16816(o[m][2 * cp + 1], pf[j2], b + 2);
        }
      }
    }
    hb_cp_async_wait<0>();
    __syncthreads();
    kt = next;
  }

  // o = O_0 / l_0 - lambda O_1 / l_1, its root mean square over the row's E values (spread over a quad's lanes)
  float inv[2][2];
#pragma unroll
  for (int m = 0; m < 2; m++)
#pragma unroll
    for (int r = 0; r < 2; r++) {
      float l = ls[m][r];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      inv[m][r] = 1.f / l;
    }
  float ss_a = 0.f, ss_b = 0.f;
#pragma unroll
  for (int i = 0; i < NT_O; i++) {
#pragma unroll
    for (int e = 0; e < 2; e++) {
      const float va = o[0][i][e] * inv[0][0] - A.lambda * (o[1][i][e] * inv[1][0]);
      const float vb = o[0][i][2 + e] * inv[0][1] - A.lambda * (o[1][i][2 + e] * inv[1][1]);
      o[0][i][e] = va;
      o[0][i][2 + e] = vb;
      ss_a = fmaf(va, va, ss_a);
      ss_b = fmaf(vb, vb, ss_b);
    }
  }
  ss_a += __shfl_xor_sync(0xffffffffu, ss_a, 1); ss_a += __shfl_xor_sync(0xffffffffu, ss_a, 2);
  ss_b += __shfl_xor_sync(0xffffffffu, ss_b, 1); ss_b += __shfl_xor_sync(0xffffffffu, ss_b, 2);
  const float f_a = rsqrtf(ss_a / (float)E + A.eps) * A.post, f_b = rsqrtf(ss_b / (float)E + A.eps) * A.post;
#pragma unroll
  for (int i = 0; i < NT_O; i++) {
    const int d = i * 8 + 2 * t;
    if (r_a < rows_here) {
      float y0 = o[0][i][0] * f_a, y1 = o[0][i][1] * f_a;
      if (A.gate) {
        const float* gp = A.gate + (size_t)(row0 + r_a) * A.ld_gate + A.gate_off + hq * E + d;
        y0 *= 1.f / (1.f + expf(-gp[0]));
        y1 *= 1.f / (1.f + expf(-gp[1]));
      }
      *(uint32_t*)(A.out + ((size_t)(row0 + r_a) * H + hq) * E + d) = hb_pack_bf16(y0, y1);
    }
    if (r_b < rows_here) {
      float y0 = o[0][i][2] * f_b, y1 = o[0][i][3] * f_b;
      if (A.gate) {
        const float* gp = A.gate + (size_t)(row0 + r_b) * A.ld_gate + A.gate_off + hq * E + d;
        y0 *= 1.f / (1.f + expf(-gp[0]));
        y1 *= 1.f / (1.f + expf(-gp[1]));
      }
      *(uint32_t*)(A.out + ((size_t)(row0 + r_b) * H + hq) * E + d) = hb_pack_bf16(y0, y1);
    }
  }
}

// ---------------------------------------------------------------------------------------
// Single rows (decode steps, short portions) on warp MMAs: the heads of a kv head are the MMA's rows.
//
// One CTA = (kv head, row, key split). The H/G query heads that share the kv head (at most 16) fill the 16 rows of one
// warp's MMA tile, so a key tile is read once for all of them; all four warps gather the split's tiles (all asked for at
// once: one trip to memory for four tiles), then each warp walks ONE tile and warp 0 joins the four. The row's
// visible tiles (kept tokens, then the window) are split RM_SPLIT_TILES a CTA, which depends on the row's position
// alone; a CTA leaves its two maps' running maximum, weight sum and value sums in a workspace and the CTA that arrives
// last at the (row, kv head) joins the splits in their order and finishes the heads (combination, head norm, gate).
// ---------------------------------------------------------------------------------------
constexpr int RM_SPLIT_TILES = 4;

struct WinRowsArgs {
  const __nv_bfloat16* q;
  const __nv_bfloat16* kc;
  const __nv_bfloat16* vc;
  const int* bt;
  int bt_stride;
  const int* row_req;
  const int* pos;
  const float* gate;
  long ld_gate;
  int gate_off;
  __nv_bfloat16* out;
  int H, G, page_size, window, keep_first;
  float scale_log2, lambda, post, eps;
  const int* q_len;      // or null: rows of requests with row_limit rows or more are left to the flash kernel
  int row_limit;
  float* part;           // [T][G][splits][2 maps][H/G][E + 2]
  int* arrived;          // [T][G], zero before and after
  int splits;
};

template <int D, int E>
__global__ void __launch_bounds__(WF_THREADS, 3) attn_window_rows_mma_kernel(WinRowsArgs A) {
  constexpr int QW = 2 * D, KS = D / 16, NT_O = E / 8, KTILE = WF_BKV * QW * 2, VTILE = WF_BKV * E * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int last;
  hb_pdl_launch();
  hb_pdl_wait();
  const int g_kv = blockIdx.x, row = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  if (A.q_len && A.q_len[A.row_req[row]] >= A.row_limit) return;
  const int H = A.H, G = A.G, HG = H / G, window = A.window;
  const int p = A.pos[row];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int keep = window > 0 ? min(A.keep_first, p + 1) : 0;
  const int last_tile = p / WF_BKV, first_win_tile = lo / WF_BKV, last_keep_tile = keep > 0 ? (keep - 1) / WF_BKV : -1;
  const int win0 = max(first_win_tile, last_keep_tile + 1), n_vis = (last_keep_tile + 1) + (last_tile - win0 + 1);
  const int n_splits = (n_vis + RM_SPLIT_TILES - 1) / RM_SPLIT_TILES;
  const int ord0 = blockIdx.z * RM_SPLIT_TILES, ord1 = min(n_vis, ord0 + RM_SPLIT_TILES);
  if (ord0 >= n_vis) return;
  auto tile_of = [&](int ord) { return ord <= last_keep_tile ? ord : win0 + (ord - (last_keep_tile + 1)); };
  const int* table = A.bt + (size_t)A.row_req[row] * A.bt_stride;
  const uint32_t sQ = hb_smem_u32(smem), sK = sQ + 16 * QW * 2, sV = sK + RM_SPLIT_TILES * KTILE;
  int* rowoff = (int*)(smem + 16 * QW * 2 + RM_SPLIT_TILES * (KTILE + VTILE));      // [RM_SPLIT_TILES][64]: a key's row in the planes, -1: not visible
  const int n_tiles = ord1 - ord0;

  // where every key of the split's tiles lies (one division and one table read a key, not one a 16-byte copy)
  for (int i = tid; i < n_tiles * WF_BKV; i += WF_THREADS) {
    const int kp = tile_of(ord0 + i / WF_BKV) * WF_BKV + (i & (WF_BKV - 1));
    const bool vis = kp <= p && (kp >= lo || kp < keep);
    rowoff[i] = vis ? (table[kp / A.page_size] * G + g_kv) * A.page_size + kp % A.page_size : -1;
  }
  for (int i = tid; i < 16 * (QW / 8); i += WF_THREADS) {      // the group's heads as rows 0 .. HG-1, the rest zero
    const int r = i / (QW / 8), c = i - r * (QW / 8);
    const uint32_t dst = sQ + wf_swz(r, c, QW * 2);
    if (r < HG) hb_cp_async16(dst, A.q + ((size_t)row * H + (size_t)g_kv * HG + r) * QW + c * 8);
    else asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
  }
  __syncthreads();
  // ALL tiles of the split are asked for at once: their trips to memory overlap, the walk then waits once
  for (int i = tid; i < n_tiles * WF_BKV * (QW / 8 + E / 8); i += WF_THREADS) {
    constexpr int CK = QW / 8, CA = QW / 8 + E / 8;
    const int kr = i / CA, c = i - kr * CA, s_ = kr / WF_BKV, r = kr & (WF_BKV - 1), off = rowoff[kr];
    const uint32_t dst = c < CK ? sK + s_ * KTILE + wf_swz(r, c, QW * 2) : sV + s_ * VTILE + wf_swz(r, c - CK, E * 2);
    if (off >= 0) hb_cp_async16(dst, c < CK ? A.kc + (size_t)off * QW + c * 8 : A.vc + (size_t)off * E + (c - CK) * 8);
    else asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
  }
  hb_cp_async_commit();
  hb_cp_async_wait<0>();
  __syncthreads();

  float o[2][NT_O][4];
#pragma unroll
  for (int m = 0; m < 2; m++)
#pragma unroll
    for (int i = 0; i < NT_O; i++) o[m][i][0] = o[m][i][1] = o[m][i][2] = o[m][i][3] = 0.f;
  float mx[2][2] = {{-INFINITY, -INFINITY}, {-INFINITY, -INFINITY}}, ls[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  const int mi = lane >> 3, lr = lane & 7;

  if (warp < n_tiles) {            // a warp a tile: the split's tiles are walked side by side
    const int it = warp;
    {
      const uint32_t tK = sK + it * KTILE, tV = sV + it * VTILE;
      const int k_base = tile_of(ord0 + it) * WF_BKV;
      const bool all_seen = k_base + WF_BKV - 1 <= p && (window <= 0 || k_base >= p - window + 1 || k_base + WF_BKV - 1 < keep);
#pragma unroll
      for (int m = 0; m < 2; m++) {
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < KS; kk++) {
          uint32_t a[4];
          hb_ldmatrix_x4(a, sQ + wf_swz((mi & 1) * 8 + lr, m * (D / 8) + kk * 2 + (mi >> 1), QW * 2));
#pragma unroll
          for (int np = 0; np < 4; np++) {
            uint32_t b[4];
            hb_ldmatrix_x4(b, tK + wf_swz(np * 16 + (mi >> 1) * 8 + lr, m * (D / 8) + kk * 2 + (mi & 1), QW * 2));
            hb_mma_16816(s[2 * np], a, b);
            hb_mma_16816(s[2 * np + 1], a, b + 2);
          }
        }
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int i = 0; i < 8; i++) {
#pragma unroll
          for (int e = 0; e < 2; e++) {
            if (!all_seen) {
              const int kp = k_base + i * 8 + 2 * t + e;
              if (!(kp <= p && (window <= 0 || kp > p - window || kp < keep))) s[i][e] = s[i][2 + e] = -INFINITY;
            }
            mx_a = fmaxf(mx_a, s[i][e]);
            mx_b = fmaxf(mx_b, s[i][2 + e]);
          }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(mx[m][0], mx_a * A.scale_log2), mn_b = fmaxf(mx[m][1], mx_b * A.scale_log2);
        const float sub_a = mn_a == -INFINITY ? 0.f : mn_a, sub_b = mn_b == -INFINITY ? 0.f : mn_b;
        const float corr_a = hb_exp2(mx[m][0] - sub_a), corr_b = hb_exp2(mx[m][1] - sub_b);
        mx[m][0] = mn_a; mx[m][1] = mn_b;
        float sum_a = 0.f, sum_b = 0.f;
        uint32_t pf[4][4];
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const float p0 = hb_exp2(s[i][0] * A.scale_log2 - sub_a), p1 = hb_exp2(s[i][1] * A.scale_log2 - sub_a);
          const float p2 = hb_exp2(s[i][2] * A.scale_log2 - sub_b), p3 = hb_exp2(s[i][3] * A.scale_log2 - sub_b);
          sum_a += p0 + p1;
          sum_b += p2 + p3;
          pf[i >> 1][(i & 1) * 2] = hb_pack_bf16(p0, p1);
          pf[i >> 1][(i & 1) * 2 + 1] = hb_pack_bf16(p2, p3);
        }
        ls[m][0] = ls[m][0] * corr_a + sum_a;
        ls[m][1] = ls[m][1] * corr_b + sum_b;
#pragma unroll
        for (int i = 0; i < NT_O; i++) { o[m][i][0] *= corr_a; o[m][i][1] *= corr_a; o[m][i][2] *= corr_b; o[m][i][3] *= corr_b; }
#pragma unroll
        for (int j2 = 0; j2 < 4; j2++) {
#pragma unroll
          for (int cp = 0; cp < NT_O / 2; cp++) {
            uint32_t b[4];
            hb_ldmatrix_x4_trans(b, tV + wf_swz(j2 * 16 + (mi & 1) * 8 + lr, cp * 2 + (mi >> 1), E * 2));
            hb_mma_16816(o[m][2 * cp], pf[j2], b);
            hb_mma_16816(o[m][2 * cp + 1], pf[j2], b + 2);
          }
        }
      }
    }
  }

  // the weight sums of a row are spread over its quad's lanes
#pragma unroll
  for (int m = 0; m < 2; m++)
#pragma unroll
    for (int r = 0; r < 2; r++) {
      ls[m][r] += __shfl_xor_sync(0xffffffffu, ls[m][r], 1);
      ls[m][r] += __shfl_xor_sync(0xffffffffu, ls[m][r], 2);
    }
  const int r_a = g, r_b = g + 8;                 // this thread's two rows (heads of the group), the same in every warp
  if (n_tiles > 1) {
    // the warps' tiles are joined in the tiles' order by warp 0, through the memory the tiles lay in
    __syncthreads();
    float* wp = (float*)(smem + 16 * QW * 2);     // [warp][2 maps][HG][E + 2]
    if (warp < n_tiles) {
#pragma unroll
      for (int m = 0; m < 2; m++) {
#pragma unroll
        for (int half = 0; half < 2; half++) {
          const int r = half ? r_b : r_a;
          if (r < HG) {
            float* pr = wp + (((size_t)warp * 2 + m) * HG + r) * (E + 2);
#pragma unroll
            for (int i = 0; i < NT_O; i++) {
              pr[i * 8 + 2 * t] = o[m][i][2 * half];
              pr[i * 8 + 2 * t + 1] = o[m][i][2 * half + 1];
            }
            if (t == 0) { pr[E] = mx[m][half]; pr[E + 1] = ls[m][half]; }
          }
        }
      }
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
      for (int m = 0; m < 2; m++) {
#pragma unroll
        for (int half = 0; half < 2; half++) {
          const int r = half ? r_b : r_a;
          if (r >= HG) continue;
          float mm = -INFINITY;
          for (int w = 0; w < n_tiles; w++) mm = fmaxf(mm, wp[(((size_t)w * 2 + m) * HG + r) * (E + 2) + E]);
          float l = 0.f;
#pragma unroll
          for (int i = 0; i < NT_O; i++) o[m][i][2 * half] = o[m][i][2 * half + 1] = 0.f;
          for (int w = 0; w < n_tiles; w++) {
            const float* pw = wp + (((size_t)w * 2 + m) * HG + r) * (E + 2);
            const float f = hb_exp2(pw[E] - mm);
            l = fmaf(pw[E + 1], f, l);
#pragma unroll
            for (int i = 0; i < NT_O; i++) {
              o[m][i][2 * half] = fmaf(pw[i * 8 + 2 * t], f, o[m][i][2 * half]);
              o[m][i][2 * half + 1] = fmaf(pw[i * 8 + 2 * t + 1], f, o[m][i][2 * half + 1]);
            }
          }
          mx[m][half] = mm;
          ls[m][half] = l;
        }
      }
    }
    __syncthreads();             // (the join of the splits below takes the same memory)
  }
  if (n_splits > 1) {
    const size_t slot = ((size_t)row * G + g_kv) * A.splits;
    if (warp == 0) {
      float* mine = A.part + (slot + blockIdx.z) * 2 * HG * (E + 2);
#pragma unroll
      for (int m = 0; m < 2; m++) {
#pragma unroll
        for (int half = 0; half < 2; half++) {
          const int r = half ? r_b : r_a;
          if (r < HG) {
            float* pr = mine + ((size_t)m * HG + r) * (E + 2);
#pragma unroll
            for (int i = 0; i < NT_O; i++) {
              pr[i * 8 + 2 * t] = o[m][i][2 * half];
              pr[i * 8 + 2 * t + 1] = o[m][i][2 * half + 1];
            }
            if (t == 0) { pr[E] = mx[m][half]; pr[E + 1] = ls[m][half]; }
          }
        }
      }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const int seen = atomicAdd(A.arrived + (size_t)row * G + g_kv, 1);
      last = seen == n_splits - 1;
      if (last) A.arrived[(size_t)row * G + g_kv] = 0;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    // join the splits in their order: first every (map, head)'s maximum and weight sum, then the value sums, a thread an
    // element, the splits' values asked for eight at a time (one trip to L2 for eight splits, not one a split)
    const float* all = A.part + slot * 2 * HG * (E + 2);
    float* joined = (float*)smem;                      // [2 * HG][E + 2]; the walk is over, the tiles' memory is free
    const size_t zs = (size_t)2 * HG * (E + 2);
    for (int idx = tid; idx < 2 * HG; idx += WF_THREADS) {
      const float* pm = all + (size_t)idx * (E + 2) + E;
      float mm = -INFINITY;
      for (int z0 = 0; z0 < n_splits; z0 += 8) {
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; k++) v[k] = z0 + k < n_splits ? __ldcg(pm + (z0 + k) * zs) : -INFINITY;
#pragma unroll
        for (int k = 0; k < 8; k++) mm = fmaxf(mm, v[k]);
      }
      float l = 0.f;
      for (int z0 = 0; z0 < n_splits; z0 += 8) {
        float v[8], w[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
          v[k] = z0 + k < n_splits ? __ldcg(pm + (z0 + k) * zs) : -INFINITY;
          w[k] = z0 + k < n_splits ? __ldcg(pm + 1 + (z0 + k) * zs) : 0.f;
        }
#pragma unroll
        for (int k = 0; k < 8; k++) l = fmaf(w[k], hb_exp2(v[k] - mm), l);
      }
      joined[idx * (E + 2) + E] = mm;
      joined[idx * (E + 2) + E + 1] = l;
    }
    __syncthreads();
    for (int idx = tid; idx < 2 * HG * E; idx += WF_THREADS) {
      const int mr = idx / E, e = idx - mr * E;
      const float* pe = all + (size_t)mr * (E + 2);
      const float mm = joined[mr * (E + 2) + E];
      float acc = 0.f;
      for (int z0 = 0; z0 < n_splits; z0 += 8) {
        float v[8], w[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
          v[k] = z0 + k < n_splits ? __ldcg(pe + e + (z0 + k) * zs) : 0.f;
          w[k] = z0 + k < n_splits ? __ldcg(pe + E + (z0 + k) * zs) : -INFINITY;
        }
#pragma unroll
        for (int k = 0; k < 8; k++) acc = fmaf(v[k], hb_exp2(w[k] - mm), acc);
      }
      joined[mr * (E + 2) + e] = acc;
    }
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int m = 0; m < 2; m++) {
#pragma unroll
      for (int half = 0; half < 2; half++) {
        const int r = half ? r_b : r_a;
        if (r >= HG) continue;
        const float* jr = joined + (m * HG + r) * (E + 2);
#pragma unroll
        for (int i = 0; i < NT_O; i++) {
          o[m][i][2 * half] = jr[i * 8 + 2 * t];
          o[m][i][2 * half + 1] = jr[i * 8 + 2 * t + 1];
        }
        ls[m][half] = jr[E + 1];
      }
    }
  } else if (warp != 0) {
    return;
  }
  // warp 0: o = O_0 / l_0 - lambda O_1 / l_1, head norm over the row's E values (a quad's lanes), post, gate
  float ss_a = 0.f, ss_b = 0.f;
  const float i0a = 1.f / ls[0][0], i1a = 1.f / ls[1][0], i0b = 1.f / ls[0][1], i1b = 1.f / ls[1][1];
#pragma unroll
  for (int i = 0; i < NT_O; i++) {
#pragma unroll
    for (int e = 0; e < 2; e++) {
      const float va = o[0][i][e] * i0a - A.lambda * (o[1][i][e] * i1a);
      const float vb = o[0][i][2 + e] * i0b - A.lambda * (o[1][i][2 + e] * i1b);
      o[0][i][e] = va;
      o[0][i][2 + e] = vb;
      ss_a = fmaf(va, va, ss_a);
      ss_b = fmaf(vb, vb, ss_b);
    }
  }
  ss_a += __shfl_xor_sync(0xffffffffu, ss_a, 1); ss_a += __shfl_xor_sync(0xffffffffu, ss_a, 2);
  ss_b += __shfl_xor_sync(0xffffffffu, ss_b, 1); ss_b += __shfl_xor_sync(0xffffffffu, ss_b, 2);
  const float f_a = rsqrtf(ss_a / (float)E + A.eps) * A.post, f_b = rsqrtf(ss_b / (float)E + A.eps) * A.post;
#pragma unroll
  for (int half = 0; half < 2; half++) {
    const int r = half ? r_b : r_a;
    if (r >= HG) continue;
    const float f = half ? f_b : f_a;
    const size_t head = (size_t)row * H + (size_t)g_kv * HG + r;
#pragma unroll
    for (int i = 0; i < NT_O; i++) {
      const int d = i * 8 + 2 * t;
      float y0 = o[0][i][2 * half] * f, y1 = o[0][i][2 * half + 1] * f;
      if (A.gate) {
        const float* gp = A.gate + (size_t)row * A.ld_gate + A.gate_off + ((size_t)g_kv * HG + r) * E + d;
        y0 *= 1.f / (1.f + expf(-gp[0]));
        y1 *= 1.f / (1.f + expf(-gp[1]));
      }
      *(uint32_t*)(A.out + head * E + d) = hb_pack_bf16(y0, y1);
    }
  }
}

HB_EXPORT int hb_attn_window_rows_mma_supported(int H, int G, int D, int E, int M) {
  return M == 2 && G > 0 && H % G == 0 && H / G <= 16 && (D == 32 || D == 64 || D == 128) && (E == 64 || E == 128);
}
HB_EXPORT int hb_attn_window_rows_mma_splits(int window, int keep_first, int max_pos) {
  const int tiles = window > 0 ? min((window + WF_BKV - 1) / WF_BKV + 1 + (keep_first + WF_BKV - 1) / WF_BKV, max_pos / WF_BKV + 1)
                               : max_pos / WF_BKV + 1;
  return (tiles + RM_SPLIT_TILES - 1) / RM_SPLIT_TILES;
}
HB_EXPORT long hb_attn_window_rows_mma_workspace(int T, int H, int G, int E, int window, int keep_first, int max_pos) {
  const int sp = hb_attn_window_rows_mma_splits(window, keep_first, max_pos);
  return sp <= 1 ? 0 : (long)T * G * sp * 2 * (H / G) * (E + 2);
}

template <int D, int E>
static int rm_launch(const WinRowsArgs& A, dim3 grid, cudaStream_t s) {
  const size_t smem = (size_t)16 * 2 * D * 2 + RM_SPLIT_TILES * ((size_t)WF_BKV * 2 * D * 2 + (size_t)WF_BKV * E * 2 + WF_BKV * sizeof(int));
  auto kern = attn_window_rows_mma_kernel<D, E>;
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) HB_FAIL("hb_attn_window_rows_mma: %s", cudaGetErrorString(e));
    configured = true;
  }
  hb_launch(kern, grid, WF_THREADS, smem, s, A);
  return 0;
}

// q [T, H, 2 D], out [T, H, E] bf16; planes as for hb_attn_window_flash; per row its request and position. max_pos: the
// largest position among the rows (bounds the key splits). part / arrived: see hb_attn_window_rows_mma_workspace.
HB_EXPORT int hb_attn_window_rows_mma(const void* q, const void* kc, const void* vc, const int* bt, int bt_stride,
                                      const int* row_req, const int* pos, const float* gate, long ld_gate, int gate_off,
                                      void* out, int T, int H, int G, int D, int E, int page_size, int window, int keep_first,
                                      float scale, float lambda, float post, float eps, const int* q_len, int row_limit,
                                      float* part, long part_floats, int* arrived, int max_pos, cudaStream_t s) {
  if (T <= 0) return 0;
  if (!hb_attn_window_rows_mma_supported(H, G, D, E, 2)) HB_FAIL("hb_attn_window_rows_mma: %d/%d heads of %d/%d are not supported", H, G, D, E);
  if (T > 65535) HB_FAIL("hb_attn_window_rows_mma: %d rows are beyond the grid limit", T);
  if (((uintptr_t)q | (uintptr_t)kc | (uintptr_t)vc | (uintptr_t)out) & 15) HB_FAIL("hb_attn_window_rows_mma: q, planes and out must be 16-byte aligned");
  const int splits = hb_attn_window_rows_mma_splits(window, keep_first, max_pos);
  if (splits > 1 && (!part || !arrived || part_floats < hb_attn_window_rows_mma_workspace(T, H, G, E, window, keep_first, max_pos)))
    HB_FAIL("hb_attn_window_rows_mma: %d key splits a row need a workspace and counters", splits);
  if (splits > 65535) HB_FAIL("hb_attn_window_rows_mma: %d key splits are beyond the grid limit", splits);
  WinRowsArgs A{(const __nv_bfloat16*)q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, bt, bt_stride, row_req, pos, gate, ld_gate,
                gate_off, (__nv_bfloat16*)out, H, G, page_size, window, keep_first, scale * 1.4426950408889634f, lambda, post, eps,
                q_len, row_limit, part, arrived, splits};
  const dim3 grid(G, T, splits);
  int r = -1;
  if (D == 32 && E == 64) r = rm_launch<32, 64>(A, grid, s);
  else if (D == 32 && E == 128) r = rm_launch<32, 128>(A, grid, s);
  else if (D == 64 && E == 64) r = rm_launch<64, 64>(A, grid, s);
  else if (D == 64 && E == 128) r = rm_launch<64, 128>(A, grid, s);
  else if (D == 128 && E == 64) r = rm_launch<128, 64>(A, grid, s);
  else if (D == 128 && E == 128) r = rm_launch<128, 128>(A, grid, s);
  if (r) return r;
  HB_CHECK_LAUNCH("hb_attn_window_rows_mma");
  return 0;
}

HB_EXPORT int hb_attn_window_flash_supported(int H, int G, int D, int E, int M) {
  return M == 2 && G > 0 && H % G == 0 && (D == 32 || D == 64 || D == 128) && (E == 64 || E == 128);
}

template <int D, int E>
static int wf_launch(const WinFlashArgs& A, dim3 grid, cudaStream_t s) {
  const size_t smem = (size_t)WF_BQ * 2 * D * 2 + 2 * ((size_t)WF_BKV * 2 * D * 2 + (size_t)WF_BKV * E * 2);
  auto kern = attn_window_flash_kernel<D, E>;
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) HB_FAIL("hb_attn_window_flash: %s", cudaGetErrorString(e));
    configured = true;
  }
  hb_launch(kern, grid, WF_THREADS, smem, s, A);
  return 0;
}

// q [T, H, 2 D], out [T, H, E] bf16; planes [page, G, page_size, 2 D] and [..., E] bf16; per request q_start, q_len,
// ctx_len and a block table row. Requests with fewer than min_rows rows are skipped (the row kernel takes them).
HB_EXPORT int hb_attn_window_flash(const void* q, const void* kc, const void* vc, const int* bt, int bt_stride,
                                   const int* q_start, const int* q_len, const int* ctx_len, const float* gate, long ld_gate,
                                   int gate_off, void* out, int R, int max_q_len, int H, int G, int D, int E, int page_size,
                                   int window, int keep_first, float scale, float lambda, float post, float eps, int min_rows,
                                   cudaStream_t s) {
  if (R <= 0 || max_q_len <= 0) return 0;
  if (!hb_attn_window_flash_supported(H, G, D, E, 2)) HB_FAIL("hb_attn_window_flash: %d/%d heads of %d/%d are not supported", H, G, D, E);
  if (R > 65535 || max_q_len > 65535 * WF_BQ) HB_FAIL("hb_attn_window_flash: %d requests / portions of %d rows are beyond the grid limit", R, max_q_len);
  if (((uintptr_t)q | (uintptr_t)kc | (uintptr_t)vc | (uintptr_t)out) & 15) HB_FAIL("hb_attn_window_flash: q, planes and out must be 16-byte aligned");
  WinFlashArgs A{(const __nv_bfloat16*)q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, bt, bt_stride, q_start, q_len, ctx_len,
                 gate, ld_gate, gate_off, (__nv_bfloat16*)out, H, G, page_size, window, keep_first,
                 scale * 1.4426950408889634f, lambda, post, eps, min_rows};
  const dim3 grid(H, (max_q_len + WF_BQ - 1) / WF_BQ, R);
  int r = -1;
  if (D == 32 && E == 64) r = wf_launch<32, 64>(A, grid, s);
  else if (D == 32 && E == 128) r = wf_launch<32, 128>(A, grid, s);
  else if (D == 64 && E == 64) r = wf_launch<64, 64>(A, grid, s);
  else if (D == 64 && E == 128) r = wf_launch<64, 128>(A, grid, s);
  else if (D == 128 && E == 64) r = wf_launch<128, 64>(A, grid, s);
  else if (D == 128 && E == 128) r = wf_launch<128, 128>(A, grid, s);
  if (r) return r;
  HB_CHECK_LAUNCH("hb_attn_window_flash");
  return 0;
}
