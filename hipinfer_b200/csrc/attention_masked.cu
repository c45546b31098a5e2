// Attention of single rows over the paged cache with the mask, the softmax and the gate chosen by parameters.
//
// Row t at position p of its request sees key j iff j <= p and
//     mask 0 (causal):  always
//     mask 1 (window):  p - j < window or j < keep_first
//     mask 2 (chunk):   floor(j / chunk) == floor(p / chunk), chunks counted from position 0 of the sequence
// The softmax may have a sink: a number per head that joins the denominator as exp(sink), with no key and no value,
// unscaled, once. The head's result may be multiplied by sigmoid of a gate, one number per element or one per head.
// Keys are D wide and values E wide; each plane is addressed by a row stride of its own, so that the values may be
// the first E columns of the key rows (a latent that serves as both). Query head h reads kv head h / (H / G).
// Scores, the running maximum and sums, exp and the sums over values are 32-bit; the result is rounded once, into an
// output element type of its own (32-bit where a 32-bit consumer follows).
//
// One block per (kv head, row, tile of RT heads of the group): its heads are score rows over one pass through the
// visible keys, which go by in tiles of MK ABSOLUTE positions (tile i holds positions [i MK, (i + 1) MK)) with a
// running maximum and sum per score row: how a row's keys are cut depends on its position alone, never on the batch
// or on how the prompt was cut. A row with many visible tiles is split over `splits` blocks of SPLIT_TILES tiles each
// (again cut at absolute tiles); the block that arrives last at (row, kv head, head tile) joins the partial results in
// the splits' order. A key that is not visible is never read (its page may have been given back).
#include "common.cuh"

#define MK 64
constexpr int MA_THREADS = 128;
constexpr int MA_SPLIT_TILES = 8;

struct MaskedArgs {
  const void* q; long ldq;          // [T][H * D]
  const void* kc; long k_row;       // key rows: ((page * G + g) * page_size + offset) * k_row
  const void* vc; long v_row;
  const int* bt; int bt_stride;     // [R][bt_stride]
  const int* row_req;               // [T]
  const int* pos;                   // [T]
  const float* sink;                // [H] or null
  const float* gate; long ld_gate; int gate_off; int gate_mode;   // 0 none, 1 one per element, 2 one per head
  void* out; long ldo;              // [T][H * E]
  int H, G, D, E, RT, page_size;
  int mask, window, keep_first, chunk;
  float scale;
  const int* q_len; int row_limit;  // rows of requests that bring row_limit rows or more are left to another kernel
  float* part;                      // [T][G][ZT][splits][RT][E + 2]
  int* arrived;                     // [T][G][ZT] zeroed counters; the last block leaves 0
  int splits;
};

__device__ __forceinline__ void ma_range(const MaskedArgs& A, int p, int& lo, int& keep) {
  lo = 0;
  keep = 0;
  if (A.mask == 1 && A.window > 0) {
    lo = max(0, p - A.window + 1);
    keep = min(A.keep_first, p + 1);
  } else if (A.mask == 2 && A.chunk > 0) {
    lo = (p / A.chunk) * A.chunk;
  }
}

// number of key tiles a row at position p walks, and the i-th of them
__device__ __host__ __forceinline__ int ma_tile_count(int p, int lo, int keep) {
  const int last = p / MK, first_win = lo / MK, last_keep = keep > 0 ? (keep - 1) / MK : -1;
  if (first_win <= last_keep + 1) return last + 1;
  return (last_keep + 1) + (last - first_win + 1);
}
__device__ __forceinline__ int ma_tile_at(int i, int lo, int keep) {
  const int first_win = lo / MK, last_keep = keep > 0 ? (keep - 1) / MK : -1;
  if (first_win <= last_keep + 1 || i <= last_keep) return i;
  return first_win + (i - (last_keep + 1));
}

template <typename TQ, typename TC, typename TO>
__global__ void __launch_bounds__(MA_THREADS) attn_masked_rows_kernel(MaskedArgs A) {
  extern __shared__ float smem[];
  hb_pdl_launch();
  hb_pdl_wait();
  const int g = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ZT = gridDim.z / A.splits, z = blockIdx.z / A.splits, split = blockIdx.z % A.splits;
  if (A.q_len && A.q_len[A.row_req[t]] >= A.row_limit) return;
  const int H = A.H, G = A.G, D = A.D, E = A.E, HG = H / G, ps = A.page_size;
  const int r_first = z * A.RT, R = min(A.RT, HG - r_first);
  float* qs = smem;                // [RT][D]
  float* sc = qs + A.RT * D;       // [RT][MK]
  float* acc = sc + A.RT * MK;     // [RT][E]
  float* mrun = acc + A.RT * E;    // [RT]
  float* lrun = mrun + A.RT;
  float* alpha = lrun + A.RT;
  int* koff = (int*)(alpha + A.RT);  // [MK]
  __shared__ int last_flag;
  const int p = A.pos[t];
  int lo, keep;
  ma_range(A, p, lo, keep);
  const int n_tiles = ma_tile_count(p, lo, keep);
  const int i0 = split * MA_SPLIT_TILES, i1 = min(n_tiles, i0 + MA_SPLIT_TILES);
  const int n_splits_row = (n_tiles + MA_SPLIT_TILES - 1) / MA_SPLIT_TILES;     // a matter of the row's position alone
  if (split >= n_splits_row) return;
  const size_t head0 = (size_t)g * HG + r_first;
  const TQ* qrow = (const TQ*)A.q + (size_t)t * A.ldq + head0 * D;
  for (int i = tid; i < R * D; i += MA_THREADS) qs[i] = hb_to_float(qrow[i]) * A.scale;
  for (int i = tid; i < R * E; i += MA_THREADS) acc[i] = 0.f;
  if (tid < R) { mrun[tid] = -INFINITY; lrun[tid] = 0.f; }
  const int* table = A.bt + (size_t)A.row_req[t] * A.bt_stride;
  const TC* kc = (const TC*)A.kc;
  const TC* vc = (const TC*)A.vc;
  for (int it = i0; it < i1; it++) {
    const int k0 = ma_tile_at(it, lo, keep) * MK;
    __syncthreads();
    if (tid < MK) {
      const int kp = k0 + tid;
      const bool vis = kp <= p && (kp >= lo || kp < keep);
      koff[tid] = vis ? (table[kp / ps] * G + g) * ps + kp % ps : -1;
    }
    __syncthreads();
    {
      const int j = tid % MK, ko = koff[j];
      for (int r = tid / MK; r < R; r += MA_THREADS / MK) {
        float a = -INFINITY;
        if (ko >= 0) {
          const TC* kr = kc + (size_t)ko * A.k_row;
          const float* qr = qs + r * D;
          a = 0.f;
          for (int d = 0; d < D; d++) a = fmaf(qr[d], hb_to_float(kr[d]), a);
        }
        sc[r * MK + j] = a;
      }
    }
    __syncthreads();
    for (int r = warp; r < R; r += MA_THREADS / 32) {
      float m = -INFINITY;
      for (int j = lane; j < MK; j += 32) m = fmaxf(m, sc[r * MK + j]);
      m = fmaxf(hb_warp_max(m), mrun[r]);
      float l = 0.f;
      for (int j = lane; j < MK; j += 32) {
        const float e = m == -INFINITY ? 0.f : expf(sc[r * MK + j] - m);
        sc[r * MK + j] = e;
        l += e;
      }
      l = hb_warp_sum(l);
      if (lane == 0) {
        const float al = m == -INFINITY ? 1.f : expf(mrun[r] - m);
        alpha[r] = al;
        lrun[r] = fmaf(lrun[r], al, l);
        mrun[r] = m;
      }
    }
    __syncthreads();
    for (int i = tid; i < R * E; i += MA_THREADS) {
      const int r = i / E, e = i - r * E;
      float a = acc[i] * alpha[r];
      for (int j = 0; j < MK; j++) {
        const int ko = koff[j];
        if (ko >= 0) a = fmaf(sc[r * MK + j], hb_to_float(vc[(size_t)ko * A.v_row + e]), a);
      }
      acc[i] = a;
    }
  }
  __syncthreads();
  if (n_splits_row > 1) {
    // leave the partial result; the block that arrives last joins them in the splits' order
    const size_t slot = (((size_t)t * G + g) * ZT + z);
    float* mine = A.part + (slot * A.splits + split) * (size_t)A.RT * (E + 2);
    for (int i = tid; i < R * E; i += MA_THREADS) mine[(i / E) * (E + 2) + i % E] = acc[i];
    if (tid < R) { mine[tid * (E + 2) + E] = mrun[tid]; mine[tid * (E + 2) + E + 1] = lrun[tid]; }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const int n = atomicAdd(A.arrived + slot, 1);
      last_flag = n == n_splits_row - 1;
      if (last_flag) A.arrived[slot] = 0;
    }
    __syncthreads();
    if (!last_flag) return;
    __threadfence();
    const float* all = A.part + slot * A.splits * (size_t)A.RT * (E + 2);
    const size_t sstride = (size_t)A.RT * (E + 2);
    if (tid < R) {
      float m = -INFINITY;
      for (int s = 0; s < n_splits_row; s++) m = fmaxf(m, __ldcg(all + s * sstride + tid * (E + 2) + E));
      float l = 0.f;
      for (int s = 0; s < n_splits_row; s++) {
        const float ms = __ldcg(all + s * sstride + tid * (E + 2) + E);
        l = fmaf(__ldcg(all + s * sstride + tid * (E + 2) + E + 1), expf(ms - m), l);
      }
      mrun[tid] = m;
      lrun[tid] = l;
    }
    __syncthreads();
    for (int i = tid; i < R * E; i += MA_THREADS) {
      const int r = i / E, e = i - r * E;
      float a = 0.f;
      for (int s = 0; s < n_splits_row; s++) {
        const float ms = __ldcg(all + s * sstride + r * (E + 2) + E);
        a = fmaf(__ldcg(all + s * sstride + r * (E + 2) + e), expf(ms - mrun[r]), a);
      }
      acc[i] = a;
    }
    __syncthreads();
  }
  for (int r = warp; r < R; r += MA_THREADS / 32) {
    const size_t head = head0 + r;
    float m = mrun[r], l = lrun[r], f = 1.f;
    if (A.sink) {
      const float sk = A.sink[head], m2 = fmaxf(m, sk);
      f = expf(m - m2);
      l = fmaf(l, f, expf(sk - m2));
    }
    f /= l;
    float gh = 1.f;
    if (A.gate_mode == 2) gh = 1.f / (1.f + expf(-A.gate[(size_t)t * A.ld_gate + A.gate_off + head]));
    for (int e = lane; e < E; e += 32) {
      float o = acc[r * E + e] * f;
      if (A.gate_mode == 1) o *= 1.f / (1.f + expf(-A.gate[(size_t)t * A.ld_gate + A.gate_off + head * E + e]));
      else if (A.gate_mode == 2) o *= gh;
      ((TO*)A.out)[(size_t)t * A.ldo + head * E + e] = hb_from_float<TO>(o);
    }
  }
}

static size_t ma_smem(int RT, int D, int E) { return ((size_t)RT * (D + MK + E + 3) + MK) * sizeof(float); }

// heads of a group a block takes, so that its shared memory stays within `budget` bytes
static int ma_head_tile(int HG, int D, int E, size_t budget) {
  int rt = HG;
  while (rt > 1 && ma_smem(rt, D, E) > budget) rt = (rt + 1) / 2;
  return rt;
}

// An upper bound of the key splits any row at a position up to max_pos needs: a run of L visible positions touches at
// most ceil((L - 1) / MK) + 1 tiles.
static int ma_splits(int mask, int window, int keep_first, int chunk, int max_pos) {
  int worst = max_pos / MK + 1;
  if (mask == 1 && window > 0) {
    const int w = (window - 1 + MK - 1) / MK + 1 + (keep_first > 0 ? (keep_first - 1) / MK + 1 : 0);
    if (w < worst) worst = w;
  } else if (mask == 2 && chunk > 0) {
    const int w = (chunk - 1 + MK - 1) / MK + 1;
    if (w < worst) worst = w;
  }
  return (worst + MA_SPLIT_TILES - 1) / MA_SPLIT_TILES;
}

HB_EXPORT long hb_attn_masked_workspace(int T, int H, int G, int D, int E, int mask, int window, int keep_first, int chunk,
                                        int max_pos) {
  const int HG = H / G, RT = ma_head_tile(HG, D, E, 96 * 1024), ZT = (HG + RT - 1) / RT;
  const int splits = ma_splits(mask, window, keep_first, chunk, max_pos);
  if (splits <= 1) return 0;
  return (long)T * G * ZT * splits * RT * (E + 2);
}
HB_EXPORT int hb_attn_masked_counters(int T, int H, int G, int D, int E) {
  const int HG = H / G, RT = ma_head_tile(HG, D, E, 96 * 1024), ZT = (HG + RT - 1) / RT;
  return T * G * ZT;
}

HB_EXPORT int hb_attn_masked(const void* q, int q_dt, long ldq, const void* kc, long k_row, const void* vc, long v_row,
                             int c_dt, const int* bt, int bt_stride, const int* row_req, const int* pos, const float* sink,
                             const float* gate, long ld_gate, int gate_off, int gate_mode, void* out, int o_dt, long ldo,
                             int T, int H, int G, int D, int E, int page_size, int mask, int window, int keep_first,
                             int chunk, float scale, const int* q_len, int row_limit, float* part, long n_part,
                             int* arrived, int max_pos, cudaStream_t s) {
  if (T <= 0) return 0;
  if (G <= 0 || H % G) HB_FAIL("hb_attn_masked: %d heads are not a multiple of %d kv heads", H, G);
  if (T > 65535) HB_FAIL("hb_attn_masked: %d rows are beyond the grid limit", T);
  MaskedArgs A;
  A.q = q; A.ldq = ldq; A.kc = kc; A.k_row = k_row; A.vc = vc; A.v_row = v_row; A.bt = bt; A.bt_stride = bt_stride;
  A.row_req = row_req; A.pos = pos; A.sink = sink; A.gate = gate; A.ld_gate = ld_gate; A.gate_off = gate_off;
  A.gate_mode = gate ? gate_mode : 0; A.out = out; A.ldo = ldo; A.H = H; A.G = G; A.D = D; A.E = E; A.page_size = page_size;
  A.mask = mask; A.window = window; A.keep_first = keep_first; A.chunk = chunk; A.scale = scale; A.q_len = q_len;
  A.row_limit = row_limit; A.part = part; A.arrived = arrived;
  const int HG = H / G;
  A.RT = ma_head_tile(HG, D, E, 96 * 1024);
  const int ZT = (HG + A.RT - 1) / A.RT;
  A.splits = ma_splits(mask, window, keep_first, chunk, max_pos);
  if (A.splits > 1 && (!part || !arrived || n_part < (long)T * G * ZT * A.splits * A.RT * (E + 2)))
    HB_FAIL("hb_attn_masked: rows of up to %d key tiles need a workspace", A.splits * MA_SPLIT_TILES);
  if (A.splits < 1) A.splits = 1;
  const size_t smem = ma_smem(A.RT, D, E);
  if (smem > 200 * 1024) HB_FAIL("hb_attn_masked: a head of %d + %d does not fit shared memory", D, E);
  dim3 grid(G, T, ZT * A.splits);
#define MA_LAUNCH(TQ, TC, TO)                                                                                      \
  do {                                                                                                             \
    auto kern = attn_masked_rows_kernel<TQ, TC, TO>;                                                               \
    if (smem + 4096 > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
    hb_launch(kern, grid, dim3(MA_THREADS), smem, s, A);                                                           \
  } while (0)
  if (q_dt == HB_F32 && c_dt == HB_F32 && o_dt == HB_F32) MA_LAUNCH(float, float, float);
  else if (q_dt == HB_BF16 && c_dt == HB_BF16 && o_dt == HB_BF16) MA_LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  else if (q_dt == HB_BF16 && c_dt == HB_BF16 && o_dt == HB_F32) MA_LAUNCH(__nv_bfloat16, __nv_bfloat16, float);
  else HB_FAIL("hb_attn_masked: element types %d/%d/%d are not a combination it takes", q_dt, c_dt, o_dt);
#undef MA_LAUNCH
  HB_CHECK_LAUNCH("hb_attn_masked");
  return 0;
}
