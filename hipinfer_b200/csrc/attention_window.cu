// Attention over the paged cache with a sliding window that keeps the first tokens, with keys and values of widths
// of their own, and with one or two score maps per head (differential attention).
//
// Row t at position p sees key j iff j <= p and (window == 0 or p - j < window or j < keep_first). A head has M
// score maps (M = 1: ordinary attention; M = 2: differential): its query is [map 0 (D) | map 1 (D)], the keys of its
// kv head likewise, and every map is a softmax of its own over the same values (E wide). For M = 2 the head's result is
//     o = a0 - lambda * a1,   then (if asked) o / sqrt(mean(o^2) + eps) * post,
// and every result may be multiplied by sigmoid(gate[t, head, :]) on its way out. Scores, softmax, the sums over
// values, the combination and the norm are 32-bit (expf); the result is rounded once.
//
// One block per (kv head, row): the H/G heads of the kv head and their maps are R = (H/G) * M score rows over one
// pass through the keys, which go by in tiles of KT ABSOLUTE positions (tile i holds positions [i KT, (i + 1) KT)),
// with a running maximum and sum per score row: how a row's keys are cut depends on its position alone, never on
// the batch or on how the prompt was cut. Tiles without a visible key are skipped; a key that is not visible is
// never read (its page may have been given back: its block-table entry is -1).
#include "common.cuh"

#define KT 64

struct WinArgs {
  const void* q;        // [T][H * M * D]
  const void* kc;       // [page][G][page_size][M * D]
  const void* vc;       // [page][G][page_size][E]
  const int* bt;        // [R][bt_stride]
  int bt_stride;
  const int* row_req;   // [T]
  const int* pos;       // [T]
  const float* gate;    // [T][ld_gate], columns gate_off .. + H * E, or null
  long ld_gate;
  int gate_off;
  void* out;            // [T][H * E]
  int H, G, D, E, M, page_size, window, keep_first;
  float scale, lambda, post, eps;
  int norm;             // divide the head's result by its root mean square
  const int* q_len;     // [R] or null: rows of requests that bring row_limit rows or more are left to the flash kernel
  int row_limit;
  float* part;          // staged kernel, several key splits a row: [T][G][splits][R][E + 2] partial (sums, maximum, weight sum)
  int* arrived;         // [T][G] zeroed counters; the block that arrives last at a (row, kv head) joins the splits and leaves 0
  int splits;           // gridDim.z
};

template <typename TQ, typename TC>
__global__ void __launch_bounds__(128) attn_window_kernel(WinArgs A) {
  extern __shared__ float smem[];
  hb_pdl_launch();
  hb_pdl_wait();
  const int g = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (A.q_len && A.q_len[A.row_req[t]] >= A.row_limit) return;
  const int H = A.H, G = A.G, D = A.D, E = A.E, M = A.M, HG = H / G, R = HG * M, ps = A.page_size;
  float* qs = smem;              // [R][D]
  float* sc = qs + R * D;        // [R][KT]
  float* acc = sc + R * KT;      // [R][E]
  float* mrun = acc + R * E;     // [R]
  float* lrun = mrun + R;        // [R]
  float* alpha = lrun + R;       // [R]
  int* koff = (int*)(alpha + R); // [KT]: the key's row in the planes ((page * G + g) * ps + offset), -1: not visible
  const int p = A.pos[t];
  const int lo = A.window > 0 ? max(0, p - A.window + 1) : 0;
  const int keep = min(A.keep_first, p + 1);
  const TQ* qrow = (const TQ*)A.q + ((size_t)t * H + (size_t)g * HG) * M * D;
  for (int i = tid; i < R * D; i += 128) qs[i] = hb_to_float(qrow[i]) * A.scale;
  for (int i = tid; i < R * E; i += 128) acc[i] = 0.f;
  if (tid < R) { mrun[tid] = -INFINITY; lrun[tid] = 0.f; }
  const int* table = A.bt + (size_t)A.row_req[t] * A.bt_stride;
  const TC* kc = (const TC*)A.kc;
  const TC* vc = (const TC*)A.vc;
  const int last_tile = p / KT, first_win_tile = lo / KT, last_keep_tile = keep > 0 ? (keep - 1) / KT : -1;
  for (int ti = 0; ti <= last_tile; ti++) {
    if (ti > last_keep_tile && ti < first_win_tile) { ti = first_win_tile - 1; continue; }
    const int k0 = ti * KT;
    __syncthreads();             // the tile before is done with sc, koff, alpha
    if (tid < KT) {
      const int kp = k0 + tid;
      const bool vis = kp <= p && (kp >= lo || kp < keep);
      koff[tid] = vis ? (table[kp / ps] * G + g) * ps + kp % ps : -1;
    }
    __syncthreads();
    {
      const int j = tid % KT, ko = koff[j];
      for (int r = tid / KT; r < R; r += 128 / KT) {
        float a = -INFINITY;
        if (ko >= 0) {
          const TC* kr = kc + ((size_t)ko * M + (r % M)) * D;
          const float* qr = qs + r * D;
          a = 0.f;
          for (int d = 0; d < D; d++) a = fmaf(qr[d], hb_to_float(kr[d]), a);
        }
        sc[r * KT + j] = a;
      }
    }
    __syncthreads();
    for (int r = warp; r < R; r += 4) {
      float m = -INFINITY;
      for (int j = lane; j < KT; j += 32) m = fmaxf(m, sc[r * KT + j]);
      m = fmaxf(hb_warp_max(m), mrun[r]);        // finite: the tile has a visible key
      float l = 0.f;
      for (int j = lane; j < KT; j += 32) {
        const float e = expf(sc[r * KT + j] - m);
        sc[r * KT + j] = e;
        l += e;
      }
      l = hb_warp_sum(l);
      if (lane == 0) {
        const float al = expf(mrun[r] - m);      // 0 at the first tile
        alpha[r] = al;
        lrun[r] = fmaf(lrun[r], al, l);
        mrun[r] = m;
      }
    }
    __syncthreads();
    for (int i = tid; i < R * E; i += 128) {
      const int r = i / E, e = i - r * E;
      float a = acc[i] * alpha[r];
      for (int j = 0; j < KT; j++) {
        const int ko = koff[j];
        if (ko >= 0) a = fmaf(sc[r * KT + j], hb_to_float(vc[(size_t)ko * E + e]), a);
      }
      acc[i] = a;
    }
  }
  __syncthreads();
  // the heads' results: a warp per head
  for (int hg = warp; hg < HG; hg += 4) {
    const int r0 = hg * M;
    const float l0 = lrun[r0], l1 = M > 1 ? lrun[r0 + 1] : 1.f;
    float ss = 0.f;
    for (int e = lane; e < E; e += 32) {
      float o = acc[r0 * E + e] / l0;
      if (M > 1) o = o - A.lambda * (acc[(r0 + 1) * E + e] / l1);
      acc[r0 * E + e] = o;
      ss = fmaf(o, o, ss);
    }
    ss = hb_warp_sum(ss);
    const float f = A.norm ? rsqrtf(ss / (float)E + A.eps) * A.post : A.post;
    const size_t head = (size_t)t * H + (size_t)g * HG + hg;
    for (int e = lane; e < E; e += 32) {
      float o = acc[r0 * E + e] * f;
      if (A.gate) o *= 1.f / (1.f + expf(-A.gate[(size_t)t * A.ld_gate + A.gate_off + (g * HG + hg) * E + e]));
      ((TQ*)A.out)[head * E + e] = hb_from_float<TQ>(o);
    }
  }
}

// The same for a bfloat16 cache whose rows are whole 16-byte chunks (M * D and E multiples of 8) and at most 16 score
// rows: a tile's keys and values are gathered into shared memory with cp.async (16 bytes a copy, the next tile while
// this one is worked on), so that global memory is read once and in whole rows; a thread owns one key of the tile and
// every second score row (with two maps: the rows of one map), and reads its key 8 elements at a time. The arithmetic
// is that of the kernel above in the same order (the score's sum runs over d = 0 .. D-1 in one chain), so a row whose
// keys one block walks gets the same bits from either. A row with more than WS_SPLIT_TILES tiles of visible keys is
// split over several blocks (gridDim.z), each with a running maximum and sums of its own; the block that arrives last
// joins them in the splits' order and finishes the row: a serial walk of a long window is bound by the latency of one
// tile after the other, many short walks are not.
__device__ __forceinline__ void win_cp16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

constexpr int WS_SPLIT_TILES = 4;      // key tiles a block walks: a row's keys are split over blocks of this many
constexpr int WS_THREADS = 512, WS_PARTS = WS_THREADS / KT;     // 16 warps: one block fills an SM's schedulers

__global__ void __launch_bounds__(WS_THREADS) attn_window_staged_kernel(WinArgs A) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  hb_pdl_launch();
  hb_pdl_wait();
  const int g = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (A.q_len && A.q_len[A.row_req[t]] >= A.row_limit) return;
  const int H = A.H, G = A.G, D = A.D, E = A.E, M = A.M, HG = H / G, R = HG * M, ps = A.page_size;
  const int KW = M * D, KP = KW + 8;          // a key row in shared memory is 16 bytes longer: rows fall on different banks
  __nv_bfloat16* Kt = (__nv_bfloat16*)smem_raw;                 // [2][KT][KP]
  __nv_bfloat16* Vt = Kt + 2 * KT * KP;                         // [2][KT][E]
  float* qs = (float*)(Vt + 2 * KT * E);                        // [R][D]
  float* sc = qs + R * D;                                       // [R][KT]
  float* acc = sc + R * KT;                                     // [R][E]
  float* mrun = acc + R * E;
  float* lrun = mrun + R;
  float* alpha = lrun + R;
  const int p = A.pos[t];
  const int lo = A.window > 0 ? max(0, p - A.window + 1) : 0;
  const int keep = A.window > 0 ? min(A.keep_first, p + 1) : 0;
  const int* table = A.bt + (size_t)A.row_req[t] * A.bt_stride;
  const __nv_bfloat16* kc = (const __nv_bfloat16*)A.kc;
  const __nv_bfloat16* vc = (const __nv_bfloat16*)A.vc;
  const int last_tile = p / KT, first_win_tile = lo / KT, last_keep_tile = keep > 0 ? (keep - 1) / KT : -1;
  const int ck = KW / 8, cv = E / 8;

  auto load_tile = [&](int buf, int ti) {
    const int k0 = ti * KT;
    __nv_bfloat16* kd = Kt + buf * KT * KP;
    __nv_bfloat16* vd = Vt + buf * KT * E;
    for (int i = tid; i < KT * (ck + cv); i += WS_THREADS) {
      const int r = i / (ck + cv), c = i - r * (ck + cv), kp = k0 + r;
      const bool vis = kp <= p && (kp >= lo || kp < keep);
      __nv_bfloat16* dst = c < ck ? kd + r * KP + c * 8 : vd + r * E + (c - ck) * 8;
      if (vis) {
        const size_t row = ((size_t)table[kp / ps] * G + g) * ps + kp % ps;
        win_cp16((uint32_t)__cvta_generic_to_shared(dst), c < ck ? kc + row * KW + c * 8 : vc + row * E + (c - ck) * 8);
      } else {
        *(uint4*)dst = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };

  // the tiles with a visible key, in order: those of the kept tokens, then the window's; split `blockIdx.z` walks
  // WS_SPLIT_TILES of them (which tiles a split gets depends on the row's position alone)
  const int win0 = max(first_win_tile, last_keep_tile + 1), n_vis = (last_keep_tile + 1) + (last_tile - win0 + 1);
  const int n_splits = (n_vis + WS_SPLIT_TILES - 1) / WS_SPLIT_TILES;
  const int ord0 = blockIdx.z * WS_SPLIT_TILES, ord1 = min(n_vis, ord0 + WS_SPLIT_TILES);
  if (ord0 >= n_vis) return;
  auto tile_of = [&](int ord) { return ord <= last_keep_tile ? ord : win0 + (ord - (last_keep_tile + 1)); };
  int ord = ord0, ti = tile_of(ord0);
  load_tile(0, ti);
  asm volatile("cp.async.commit_group;" ::: "memory");
  const __nv_bfloat16* qrow = (const __nv_bfloat16*)A.q + ((size_t)t * H + (size_t)g * HG) * M * D;
  for (int i = tid; i < R * D; i += WS_THREADS) qs[i] = __bfloat162float(qrow[i]) * A.scale;
  for (int i = tid; i < R * E; i += WS_THREADS) acc[i] = 0.f;
  if (tid < R) { mrun[tid] = -INFINITY; lrun[tid] = 0.f; }   // (R <= 16 < WS_THREADS)

  for (int it = 0; ord < ord1; it++, ord++) {
    const int buf = it & 1;
    const int next = ord + 1 < ord1 ? tile_of(ord + 1) : -1;
    if (next >= 0) load_tile(buf ^ 1, next);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    const int k0 = ti * KT;
    {
      // thread = (key j of the tile, part): score rows part and part + WS_PARTS (with two maps both are rows of map part % 2)
      const int j = tid & (KT - 1), part = tid >> 6, kp = k0 + j;
      const bool vis = kp <= p && (kp >= lo || kp < keep);
      const __nv_bfloat16* krow = Kt + (buf * KT + j) * KP + (part % M) * D;
      float a[2] = {0.f, 0.f};
      for (int c = 0; c < D / 8; c++) {
        const uint4 raw = *(const uint4*)(krow + c * 8);
        const __nv_bfloat162* h2 = (const __nv_bfloat162*)&raw;
        float kf[8];
#pragma unroll
        for (int x = 0; x < 4; x++) { const float2 f = __bfloat1622float2(h2[x]); kf[2 * x] = f.x; kf[2 * x + 1] = f.y; }
#pragma unroll
        for (int i = 0; i < 2; i++) {
          const int r = part + WS_PARTS * i;
          if (r < R) {
            const float4* qr = (const float4*)(qs + r * D + c * 8);
            const float4 q0 = qr[0], q1 = qr[1];
            a[i] = fmaf(q0.x, kf[0], a[i]); a[i] = fmaf(q0.y, kf[1], a[i]); a[i] = fmaf(q0.z, kf[2], a[i]); a[i] = fmaf(q0.w, kf[3], a[i]);
            a[i] = fmaf(q1.x, kf[4], a[i]); a[i] = fmaf(q1.y, kf[5], a[i]); a[i] = fmaf(q1.z, kf[6], a[i]); a[i] = fmaf(q1.w, kf[7], a[i]);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const int r = part + WS_PARTS * i;
        if (r < R) sc[r * KT + j] = vis ? a[i] : -INFINITY;
      }
    }
    __syncthreads();
    for (int r = warp; r < R; r += WS_THREADS / 32) {
      float m = -INFINITY;
      for (int j = lane; j < KT; j += 32) m = fmaxf(m, sc[r * KT + j]);
      m = fmaxf(hb_warp_max(m), mrun[r]);
      float l = 0.f;
      for (int j = lane; j < KT; j += 32) {
        const float e = expf(sc[r * KT + j] - m);
        sc[r * KT + j] = e;
        l += e;
      }
      l = hb_warp_sum(l);
      if (lane == 0) {
        const float al = expf(mrun[r] - m);
        alpha[r] = al;
        lrun[r] = fmaf(lrun[r], al, l);
        mrun[r] = m;
      }
    }
    __syncthreads();
    {
      // a thread owns value column e of TWO score rows (one read of a value serves both), four keys a step; a key
      // that is not visible has weight 0 and a zeroed row of values, so it adds nothing
      const __nv_bfloat16* vt = Vt + buf * KT * E;
      const int RP = (R + 1) >> 1;
      for (int i = tid; i < RP * E; i += WS_THREADS) {
        const int rp = i / E, e = i - rp * E, r0 = 2 * rp, r1 = min(r0 + 1, R - 1);
        const float4* p0 = (const float4*)(sc + r0 * KT);
        const float4* p1 = (const float4*)(sc + r1 * KT);
        float a0 = acc[r0 * E + e] * alpha[r0], a1 = acc[r1 * E + e] * alpha[r1];
#pragma unroll 4
        for (int j4 = 0; j4 < KT / 4; j4++) {
          const float4 w0 = p0[j4], w1 = p1[j4];
          const float v0 = __bfloat162float(vt[(4 * j4) * E + e]), v1 = __bfloat162float(vt[(4 * j4 + 1) * E + e]);
          const float v2 = __bfloat162float(vt[(4 * j4 + 2) * E + e]), v3 = __bfloat162float(vt[(4 * j4 + 3) * E + e]);
          a0 = fmaf(w0.x, v0, a0); a0 = fmaf(w0.y, v1, a0); a0 = fmaf(w0.z, v2, a0); a0 = fmaf(w0.w, v3, a0);
          a1 = fmaf(w1.x, v0, a1); a1 = fmaf(w1.y, v1, a1); a1 = fmaf(w1.z, v2, a1); a1 = fmaf(w1.w, v3, a1);
        }
        acc[r0 * E + e] = a0;
        if (r1 != r0) acc[r1 * E + e] = a1;
      }
    }
    __syncthreads();
    ti = next;
  }
  if (n_splits > 1) {
    // leave this split's sums; the block that arrives last at the (row, kv head) joins all splits in their order
    __shared__ int last;
    const size_t slot = ((size_t)t * G + g) * A.splits;
    float* mine = A.part + (slot + blockIdx.z) * R * (E + 2);
    for (int i = tid; i < R * E; i += WS_THREADS) mine[(i / E) * (E + 2) + i % E] = acc[i];
    if (tid < R) { mine[tid * (E + 2) + E] = mrun[tid]; mine[tid * (E + 2) + E + 1] = lrun[tid]; }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const int seen = atomicAdd(A.arrived + (size_t)t * G + g, 1);
      last = seen == n_splits - 1;
      if (last) A.arrived[(size_t)t * G + g] = 0;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    const float* all = A.part + slot * R * (E + 2);
    // (the splits' values are asked for eight at a time: one trip to L2 for eight splits, not one a split)
    const size_t zs = (size_t)R * (E + 2);
    if (tid < R) {
      const float* pm = all + (size_t)tid * (E + 2) + E;
      float m = -INFINITY;
      for (int z0 = 0; z0 < n_splits; z0 += 8) {
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; k++) v[k] = z0 + k < n_splits ? __ldcg(pm + (z0 + k) * zs) : -INFINITY;
#pragma unroll
        for (int k = 0; k < 8; k++) m = fmaxf(m, v[k]);
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
        for (int k = 0; k < 8; k++) l = fmaf(w[k], expf(v[k] - m), l);
      }
      mrun[tid] = m;
      lrun[tid] = l;
    }
    __syncthreads();
    for (int i = tid; i < R * E; i += WS_THREADS) {
      const int r = i / E, e = i - r * E;
      const float* pe = all + (size_t)r * (E + 2);
      const float m = mrun[r];
      float a = 0.f;
      for (int z0 = 0; z0 < n_splits; z0 += 8) {
        float v[8], w[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
          v[k] = z0 + k < n_splits ? __ldcg(pe + e + (z0 + k) * zs) : 0.f;
          w[k] = z0 + k < n_splits ? __ldcg(pe + E + (z0 + k) * zs) : -INFINITY;
        }
#pragma unroll
        for (int k = 0; k < 8; k++) a = fmaf(v[k], expf(w[k] - m), a);
      }
      acc[i] = a;
    }
    __syncthreads();
  }
  for (int hg = warp; hg < HG; hg += WS_THREADS / 32) {
    const int r0 = hg * M;
    const float l0 = lrun[r0], l1 = M > 1 ? lrun[r0 + 1] : 1.f;
    float ss = 0.f;
    for (int e = lane; e < E; e += 32) {
      float o = acc[r0 * E + e] / l0;
      if (M > 1) o = o - A.lambda * (acc[(r0 + 1) * E + e] / l1);
      acc[r0 * E + e] = o;
      ss = fmaf(o, o, ss);
    }
    ss = hb_warp_sum(ss);
    const float f = A.norm ? rsqrtf(ss / (float)E + A.eps) * A.post : A.post;
    const size_t head = (size_t)t * H + (size_t)g * HG + hg;
    for (int e = lane; e < E; e += 32) {
      float o = acc[r0 * E + e] * f;
      if (A.gate) o *= 1.f / (1.f + expf(-A.gate[(size_t)t * A.ld_gate + A.gate_off + (g * HG + hg) * E + e]));
      ((__nv_bfloat16*)A.out)[head * E + e] = __float2bfloat16_rn(o);
    }
  }
}

// Key splits a row of the staged kernel can have: tiles of the kept tokens and of the window (or, without a window,
// of all positions up to max_pos), WS_SPLIT_TILES a split. Floats of workspace for T rows (0: one split, none needed).
HB_EXPORT int hb_attn_window_splits(int window, int keep_first, int max_pos) {
  const int tiles = window > 0 ? min((window + KT - 1) / KT + 1 + (keep_first + KT - 1) / KT, max_pos / KT + 1) : max_pos / KT + 1;
  return (tiles + WS_SPLIT_TILES - 1) / WS_SPLIT_TILES;
}
HB_EXPORT long hb_attn_window_workspace(int T, int H, int G, int E, int M, int window, int keep_first, int max_pos) {
  const int sp = hb_attn_window_splits(window, keep_first, max_pos);
  return sp <= 1 ? 0 : (long)T * G * sp * (H / G * M) * (E + 2);
}

HB_EXPORT int hb_attn_window(const void* q, int q_dt, const void* kc, const void* vc, int cache_dt, const int* bt,
                             int bt_stride, const int* row_req, const int* pos, const float* gate, long ld_gate,
                             int gate_off, void* out, int T, int H, int G, int D, int E, int M, int page_size, int window,
                             int keep_first, float scale, float lambda, float post, float eps, int norm, const int* q_len,
                             int row_limit, int force_plain, float* part, long part_floats, int* arrived, int max_pos,
                             cudaStream_t s) {
  if (T <= 0) return 0;
  if (G <= 0 || H % G) HB_FAIL("hb_attn_window: %d query heads are not a multiple of %d kv heads", H, G);
  if (M != 1 && M != 2) HB_FAIL("hb_attn_window: %d score maps (1 or 2)", M);
  if (q_dt != cache_dt) HB_FAIL("hb_attn_window: q and the cache must have the same element type");
  if (window < 0 || keep_first < 0) HB_FAIL("hb_attn_window: window %d, kept first tokens %d", window, keep_first);
  if (T > 65535) HB_FAIL("hb_attn_window: %d rows are beyond the grid limit", T);
  const int R = H / G * M;
  const size_t smem = ((size_t)R * (D + KT + E + 3) + KT) * sizeof(float);
  if (smem > 200 * 1024) HB_FAIL("hb_attn_window: %d score rows of %d + %d need %zu bytes of shared memory", R, D, E, smem);
  WinArgs A{q, kc, vc, bt, bt_stride, row_req, pos, gate, ld_gate, gate_off, out, H, G, D, E, M, page_size, window, keep_first,
            scale, lambda, post, eps, norm, q_len, row_limit, part, arrived, 1};
  const size_t staged = (size_t)2 * KT * (M * D + 8 + E) * 2 + ((size_t)R * (D + KT + E + 3)) * sizeof(float);
  if (q_dt == HB_BF16 && !force_plain && (M * D) % 8 == 0 && E % 8 == 0 && D % 8 == 0 && R <= 16 && staged <= 200 * 1024 &&
      !(((uintptr_t)kc | (uintptr_t)vc) & 15)) {
    if (staged > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(attn_window_staged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)staged);
      if (e != cudaSuccess) HB_FAIL("hb_attn_window: %s", cudaGetErrorString(e));
    }
    A.splits = hb_attn_window_splits(window, keep_first, max_pos);
    if (A.splits > 1 && (!part || !arrived || part_floats < hb_attn_window_workspace(T, H, G, E, M, window, keep_first, max_pos)))
      HB_FAIL("hb_attn_window: %d key splits a row need a workspace and counters", A.splits);
    if (A.splits > 65535) HB_FAIL("hb_attn_window: %d key splits are beyond the grid limit", A.splits);
    hb_launch(attn_window_staged_kernel, dim3(G, T, A.splits), WS_THREADS, staged, s, A);
    HB_CHECK_LAUNCH("hb_attn_window");
    return 0;
  }
  HB_DISPATCH_1(q_dt, "hb_attn_window", {
    auto kern = attn_window_kernel<TA, TA>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) HB_FAIL("hb_attn_window: %s", cudaGetErrorString(e));
    }
    hb_launch(kern, dim3(G, T), 128, smem, s, A);
  });
  HB_CHECK_LAUNCH("hb_attn_window");
  return 0;
}
