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

HB_EXPORT int hb_attn_window(const void* q, int q_dt, const void* kc, const void* vc, int cache_dt, const int* bt,
                             int bt_stride, const int* row_req, const int* pos, const float* gate, long ld_gate,
                             int gate_off, void* out, int T, int H, int G, int D, int E, int M, int page_size, int window,
                             int keep_first, float scale, float lambda, float post, float eps, int norm, const int* q_len,
                             int row_limit, cudaStream_t s) {
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
            scale, lambda, post, eps, norm, q_len, row_limit};
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
