// All decoder layers of a single-token step in ONE persistent kernel (included by attention_mma.cu,
// whose head-size helpers it uses).
//
// At one to eight sequences a decode step is weight streaming broken up by dependencies: every
// projection needs all of the one before it. As separate launches each of the five kernels of a layer
// starts its memory pipeline from empty and ends it with a tail. Here one block per SM stays resident
// for the whole step; the blocks meet at a grid-wide barrier between phases, and each thread keeps a
// private ring of weight copies (cp.async) that runs ahead of the arithmetic, across phases and layers:
// weights are written by nobody, so the copies for the next projection are in flight while the block
// waits at the barrier.
//
// A layer is the pre-norm block of the reference (engine/model.py:284-303 of
// willzeng274/kernel-rush-kawk): x += Wo attention(rope(norm_qk(Wqkv rmsnorm(x)))), x += Wdown
// swiglu(Wgu rmsnorm(x)), with the rounding points of its bfloat16 kernels (gemm.py:22-51,108-113,
// rope.py:19-30, attention.py:104-122): every projection's output is rounded to bfloat16, the
// residual sum is rounded, the normalised value is rounded before the gain.
//
// Phases of a layer (a grid barrier after each):
//   1 s = round(x + branch), h = rmsnorm(s) in every block (shared memory); qkv = h Wqkv^T
//   2 per (sequence, kv head, key split): q/k norm, rotation, cache write, attention over the split's
//     pages; the last split to finish merges the partial results
//   3 branch = attn Wo^T
//   4 s = round(x + branch), h = rmsnorm(s); act = swiglu(h Wgate^T, h Wup^T)
//   5 branch = act Wdown^T
// The kernel ends with x and the last branch pending, as the layer-by-layer path does.
//
// Measured on a B200 at the Qwen3-4B layer sizes, context 1,024: 3.5 ms a step at one sequence and 4.5 ms
// at eight, against 2.1 and 2.2 ms for the layer-by-layer path, so the library does not use it unless asked
// (KRK_DECODE_PROGRAM=1). Per layer (95 us): grid barriers 5 x 3.5 us, the two norms 2.3 us each, attention
// 8 us, and the projections at 2 to 4.5 TB/s: with eight warps per SM the chain wait -> fragment load ->
// two dependent MMAs -> address arithmetic -> copy issue of one warp is not hidden by the others, and the
// look-ahead queue of batch rows in registers stalls on its own moves. The separate launches overlap
// their boundaries better (programmatic dependent launch, 0.7 us a boundary) than a grid barrier does.
//
// A projection is cut into chunks of 16 weight rows x 32 k (1 KB); the chunks of a phase, in row-tile
// order, are dealt to the blocks in equal contiguous ranges, and the warps of a block take every
// eighth chunk of its range. A row tile that straddles two blocks is summed by the second of the
// two to arrive (head part + tail part, in that order: results do not depend on who came second).
#pragma once

namespace decode_layers {

constexpr int WARPS = 8;
constexpr int NTHREADS = WARPS * 32;
constexpr int RING = 16;         // chunk steps in flight per thread (2 x 16 bytes each)
constexpr int CHUNK_K = 32;
constexpr int BPIPE = 4;         // steps of look-ahead for batch rows read from global memory
constexpr unsigned long long BARRIER_LIMIT_NS = 200ull * 1000 * 1000;

struct Layer {
  const bf16* w_qkv;   // [(HQ + 2 HKV) D, H]
  const bf16* w_o;     // [H, HQ D]
  const bf16* w_gu;    // [2 I, H]: gate rows, then up rows
  const bf16* w_down;  // [H, I]
  const void* g_attn;  // [H]
  const void* g_mlp;   // [H]
  const void* g_q;     // [D] or null
  const void* g_k;     // [D] or null
  bf16* k_cache;
  bf16* v_cache;
  const int* table;
  int width, window;
  float eps_attn, eps_mlp, eps_qk;
  int gains_f32;
};

struct Args {
  const Layer* layers;
  int n_layers, M, H, HQ, HKV, I;
  bf16* x0;            // [M][H] residual stream at entry; the stream alternates between x0 and x1
  bf16* x1;
  bf16* qkv;           // [M][(HQ + 2 HKV) D]
  bf16* attn;          // [M][HQ D]
  bf16* branch;        // [M][H]
  bf16* act;           // [M][I]
  float* part;         // [2][tiles][256]: head and tail parts of straddling row tiles (two values per thread for gate/up)
  int* tile_flags;     // [tiles], zero
  float* att_part;     // [M HKV splits][16][D + 2]
  int* att_flags;      // [M HKV], zero
  unsigned int* barrier;  // zero at launch
  const bf16* cos_t;
  const bf16* sin_t;
  int n_pos;
  const int* seq_slot;
  const int* seq_start;
  float scale_log2;
  int splits;
  int* error;
};

enum Phase { QKV = 0, OUT = 1, GATE_UP = 2, DOWN = 3 };

// Geometry of a projection phase for one block.
struct Geo {
  const bf16* W;
  int K, N;       // N: output features (I for gate/up)
  int cpt;        // chunks per row tile (twice K/32 for gate/up: the gate chunks, then the up chunks)
  int tiles;
  int begin, end; // this block's chunk range
  int up_rows;    // row offset of the up half (gate/up), else 0
};

__device__ __forceinline__ Geo geometry(const Args& a, int layer, int phase) {
  const Layer& d = a.layers[layer];
  Geo g;
  g.up_rows = 0;
  switch (phase) {
    case QKV: g.W = d.w_qkv; g.K = a.H; g.N = (a.HQ + 2 * a.HKV) * D; break;
    case OUT: g.W = d.w_o; g.K = a.HQ * D; g.N = a.H; break;
    case GATE_UP: g.W = d.w_gu; g.K = a.H; g.N = a.I; g.up_rows = a.I; break;
    default: g.W = d.w_down; g.K = a.I; g.N = a.H; break;
  }
  g.cpt = (g.K / CHUNK_K) * (phase == GATE_UP ? 2 : 1);
  g.tiles = g.N / 16;
  const long long total = (long long)g.tiles * g.cpt;
  g.begin = (int)(total * blockIdx.x / gridDim.x);
  g.end = (int)(total * (blockIdx.x + 1) / gridDim.x);
  return g;
}

// A warp's walk over its chunks: L = begin + warp, + 8, ... inside a phase; `hop` moves on to the next
// projection (of the next layer after DOWN). The copy side hops by itself, the arithmetic side is
// re-entered phase by phase; both enumerate the same steps.
struct Walk {
  Geo g;
  int layer, phase;
  int L, tile, kc;
  bool done;

  __device__ __forceinline__ void enter(const Args& a, int warp) {
    for (;;) {
      if (layer >= a.n_layers) { done = true; return; }
      g = geometry(a, layer, phase);
      L = g.begin + warp;
      if (L < g.end) break;
      next_phase();
    }
    tile = L / g.cpt;
    kc = L % g.cpt;
    done = false;
  }
  __device__ __forceinline__ void next_phase() {
    if (++phase == 4) { phase = 0; ++layer; }
  }
  __device__ __forceinline__ void step() {
    L += WARPS;
    kc += WARPS;
    while (kc >= g.cpt) { kc -= g.cpt; ++tile; }
  }
  // source of this lane's two 16-byte pieces of the chunk: rows tile*16 + g and + 8, k = 32 kc + 8 t
  __device__ __forceinline__ const bf16* source(int gq, int t) const {
    const int half_cpt = g.up_rows ? g.cpt / 2 : g.cpt;
    const int up = kc >= half_cpt ? 1 : 0;
    const int k = kc - up * half_cpt;
    return g.W + (size_t)(up * g.up_rows + tile * 16 + gq) * g.K + (size_t)k * CHUNK_K + 8 * t;
  }
};

struct Shared {
  uint4* ring;     // [RING][2][NTHREADS]
  float* red;      // [2][WARPS][2][128]
  bf16* xs;        // [8][pitch] normalised rows; the attention phase reuses the space
  int* word;       // a few words for broadcasts
};

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// All blocks of the grid meet here. False if the wait ran out or another block reported an error.
__device__ __forceinline__ bool grid_barrier(const Args& a, unsigned int& generation, int* word) {
  __syncthreads();
  if (threadIdx.x == 0) {
    ++generation;
    const unsigned int target = generation * gridDim.x;
    __threadfence();
    atomicAdd(a.barrier, 1u);
    int ok = 1;
    unsigned long long t0 = 0;
    for (unsigned int i = 1;; ++i) {
      unsigned int v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(a.barrier) : "memory");
      if (v >= target) break;
      if ((i & 63u) == 0) {
        if (*reinterpret_cast<volatile int*>(a.error) != 0) { ok = 0; break; }
        const unsigned long long now = now_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > BARRIER_LIMIT_NS) { atomicExch(a.error, 20); ok = 0; break; }
      }
    }
    __threadfence();
    word[0] = ok;
  }
  __syncthreads();
  const bool ok = word[0] != 0;
  __syncthreads();
  return ok;
}

// s = round(x + branch) (written to x_out by block 0), h = round(gain * round(s * rsqrt(mean(s^2) + eps)))
// into shared memory, for every batch row, by all threads of the block.
__device__ __forceinline__ void norm_rows(const Args& a, const Shared& sh, const bf16* x, const bf16* branch, bf16* x_out,
                                          const void* gain, int gain_f32, float eps, int pitch) {
  const int H = a.H, M = a.M, H8 = H / 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* partial = sh.red;  // [8][WARPS]
  float sq[8];
#pragma unroll
  for (int m = 0; m < 8; ++m) sq[m] = 0.f;
  for (int c = threadIdx.x; c < H8; c += NTHREADS) {
    const int k = c * 8;
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      if (m < M) {
        uint4 xv = __ldcg(reinterpret_cast<const uint4*>(x + (size_t)m * H + k));
        __nv_bfloat162* xp = reinterpret_cast<__nv_bfloat162*>(&xv);
        if (branch) {
          const uint4 bv = __ldcg(reinterpret_cast<const uint4*>(branch + (size_t)m * H + k));
          const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
          for (int j = 0; j < 4; ++j) xp[j] = __hadd2_rn(xp[j], bp[j]);
        }
        if (blockIdx.x == 0 && x_out) __stcg(reinterpret_cast<uint4*>(x_out + (size_t)m * H + k), xv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float lo = __low2float(xp[j]), hi = __high2float(xp[j]);
          sq[m] += lo * lo + hi * hi;
        }
        *reinterpret_cast<uint4*>(sh.xs + (size_t)m * pitch + k) = xv;
      }
    }
  }
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    const float v = warp_sum(sq[m]);
    if (lane == 0) partial[m * WARPS + warp] = v;
  }
  __syncthreads();
  for (int m = 0; m < M; ++m) {
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) total += partial[m * WARPS + w];
    const float r = rsqrtf(total / (float)H + eps);
    bf16* dst = sh.xs + (size_t)m * pitch;
    for (int c = threadIdx.x; c < H8; c += NTHREADS) {
      const int k = c * 8;
      uint4 xv = *reinterpret_cast<uint4*>(dst + k);
      __nv_bfloat162* xp = reinterpret_cast<__nv_bfloat162*>(&xv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 n = __floats2bfloat162_rn(__low2float(xp[j]) * r, __high2float(xp[j]) * r);
        if (gain_f32) {
          const float* gp = reinterpret_cast<const float*>(gain) + k + 2 * j;
          xp[j] = __floats2bfloat162_rn(gp[0] * __low2float(n), gp[1] * __high2float(n));
        } else {
          xp[j] = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(reinterpret_cast<const bf16*>(gain) + k + 2 * j), n);
        }
      }
      *reinterpret_cast<uint4*>(dst + k) = xv;
    }
  }
  __syncthreads();
}

__device__ __forceinline__ float silu_round(float gate) { return round_to<bf16>(gate / (1.0f + expf(-gate))); }

// One projection phase. B_SMEM: the batch rows are the normalised rows in shared memory; else they are
// read from global memory (b_src [M][K], written by other blocks in an earlier phase), a few steps ahead.
// GU: gate and up accumulate side by side and the tile's output is swiglu(gate, up).
template <bool B_SMEM, bool GU>
__device__ __forceinline__ void project(const Args& a, const Shared& sh, Walk& con, Walk& iss, unsigned int& n_steps,
                                        int& red_buf, const bf16* b_src, bf16* out, int pitch, int layer, int phase) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gq = lane >> 2, t = lane & 3;
  con.layer = layer;
  con.phase = phase;
  con.g = geometry(a, layer, phase);
  con.L = con.g.begin + warp;
  con.tile = con.L / con.g.cpt;
  con.kc = con.L % con.g.cpt;
  const Geo& g = con.g;
  if (g.begin >= g.end) return;
  const int half_cpt = GU ? g.cpt / 2 : g.cpt;
  const bool row_on = gq < a.M;

  // look-ahead queue of this lane's batch-row pieces (global source only)
  uint4 bq[BPIPE];
  auto fetch_b = [&](int L) -> uint4 {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row_on && L < g.end) v = __ldcg(reinterpret_cast<const uint4*>(b_src + (size_t)gq * g.K + (size_t)(L % g.cpt) * CHUNK_K + 8 * t));
    return v;
  };
  if (!B_SMEM) {
#pragma unroll
    for (int i = 0; i < BPIPE; ++i) bq[i] = fetch_b(con.L + i * WARPS);
  }

  for (int tile = g.begin / g.cpt; tile * g.cpt < g.end; ++tile) {
    const int t_begin = tile * g.cpt, t_end = t_begin + g.cpt;
    const int p_end = min(g.end, t_end);
    const bool from_start = g.begin <= t_begin, to_end = g.end >= t_end;
    float acc[GU ? 2 : 1][4];
#pragma unroll
    for (int s = 0; s < (GU ? 2 : 1); ++s)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[s][c] = 0.f;

    while (con.L < p_end) {
      cp_async_wait<RING - 1>();
      const uint4* slot = sh.ring + (size_t)(n_steps % RING) * 2 * NTHREADS + threadIdx.x;
      const uint4 w0 = slot[0], w1 = slot[NTHREADS];
      const int up = (GU && con.kc >= half_cpt) ? 1 : 0;
      const int k = con.kc - up * half_cpt;
      uint4 xb;
      if (B_SMEM) {
        xb = row_on ? *reinterpret_cast<const uint4*>(sh.xs + (size_t)gq * pitch + (size_t)k * CHUNK_K + 8 * t) : make_uint4(0, 0, 0, 0);
      } else {
        xb = bq[0];
#pragma unroll
        for (int i = 0; i + 1 < BPIPE; ++i) bq[i] = bq[i + 1];
        bq[BPIPE - 1] = fetch_b(con.L + BPIPE * WARPS);
      }
      if (GU && up) {
        mma_bf16_16816(acc[GU ? 1 : 0], w0.x, w1.x, w0.y, w1.y, xb.x, xb.y);
        mma_bf16_16816(acc[GU ? 1 : 0], w0.z, w1.z, w0.w, w1.w, xb.z, xb.w);
      } else {
        mma_bf16_16816(acc[0], w0.x, w1.x, w0.y, w1.y, xb.x, xb.y);
        mma_bf16_16816(acc[0], w0.z, w1.z, w0.w, w1.w, xb.z, xb.w);
      }
      con.step();
      // refill the slot just read with the copy side's next chunk
      if (!iss.done) {
        uint4* dst = sh.ring + (size_t)(n_steps % RING) * 2 * NTHREADS + threadIdx.x;
        const bf16* src = iss.source(gq, t);
        cp_async_16(dst, src);
        cp_async_16(dst + NTHREADS, src + (size_t)8 * iss.g.K);
        iss.step();
        if (iss.L >= iss.g.end) { iss.next_phase(); iss.enter(a, warp); }
      }
      cp_async_commit();
      ++n_steps;
    }

    // the block's sum for this tile (or its part of it), warps in a fixed order
    red_buf ^= 1;
    float* red = sh.red + (size_t)red_buf * WARPS * 2 * 128;
#pragma unroll
    for (int s = 0; s < (GU ? 2 : 1); ++s)
#pragma unroll
      for (int c = 0; c < 4; ++c) red[((size_t)warp * 2 + s) * 128 + c * 32 + lane] = acc[s][c];
    __syncthreads();
    float v = 0.f, v2 = 0.f;
    const int r = threadIdx.x >> 3, m = threadIdx.x & 7;  // for threads 0..127: weight row in the tile, batch row
    if (threadIdx.x < 128) {
      const int src_lane = (r % 8) * 4 + m / 2, reg = (r / 8) * 2 + (m & 1);
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        v += red[((size_t)w * 2 + 0) * 128 + reg * 32 + src_lane];
        if (GU) v2 += red[((size_t)w * 2 + 1) * 128 + reg * 32 + src_lane];
      }
    }
    bool write = from_start && to_end;
    if (!write) {
      // a tile shared with the neighbouring block: leave this part, and if the other part is there, add them
      const int mine = from_start ? 0 : 1;
      float* my_part = a.part + ((size_t)mine * g.tiles + tile) * 256;
      const float* their_part = a.part + ((size_t)(1 - mine) * g.tiles + tile) * 256;
      if (threadIdx.x < 128) {
        __stcg(my_part + threadIdx.x, v);
        if (GU) __stcg(my_part + 128 + threadIdx.x, v2);
      }
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        const int old = atomicAdd(a.tile_flags + tile, 1);
        if (old == 1) { __threadfence(); a.tile_flags[tile] = 0; }
        sh.word[1] = old;
      }
      __syncthreads();
      write = sh.word[1] == 1;
      if (write && threadIdx.x < 128) {
        const float other = __ldcg(their_part + threadIdx.x);
        v = mine == 0 ? v + other : other + v;  // head part + tail part
        if (GU) {
          const float other2 = __ldcg(their_part + 128 + threadIdx.x);
          v2 = mine == 0 ? v2 + other2 : other2 + v2;
        }
      }
    }
    if (write && threadIdx.x < 128 && m < a.M) {
      const int n = tile * 16 + r;
      if (GU) v = silu_round(round_to<bf16>(v)) * round_to<bf16>(v2);
      out[(size_t)m * g.N + n] = __float2bfloat16_rn(v);
    }
  }
}

// ---- the attention phase -------------------------------------------------------------------------
// Work item = (sequence, kv head, key split); warps 0..3 compute it as the single-token kernel of this
// file does, the last split of a (sequence, kv head) to finish merges all of them.
constexpr int ATT_THREADS = 128;
constexpr int PAGE_PIECES = KRK_PAGE * (D / 8);               // 16-byte pieces of a page of one kv head
constexpr int PIECES_PER_THREAD = (PAGE_PIECES + ATT_THREADS - 1) / ATT_THREADS;
constexpr int RP = D + 2;

struct AttShared {
  bf16* page;      // [2][64][DP]: keys, values of the current page; later the warps' partial results
  bf16* q_s;       // [16][DP]
  bf16* kv_new;    // [2][D]
  bf16* rows;      // [18][D] the new token's raw q rows (up to 16), k row, v row
};

__device__ __forceinline__ void attention_item(const Args& a, const Layer& d, const AttShared& as, int* word, int item) {
  const int splits = a.splits;
  const int split = item % splits, kh = (item / splits) % a.HKV, seq = item / (splits * a.HKV);
  const int G = a.HQ / a.HKV;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const bool worker = threadIdx.x < ATT_THREADS;
  int pos = a.seq_start[seq];
  const int slot = a.seq_slot[seq];
  if (pos < 0 || pos >= a.n_pos) {
    if (threadIdx.x == 0) atomicExch(a.error, 2);
    pos = max(0, min(pos, a.n_pos - 1));
  }
  const int lo = d.window > 0 ? max(0, pos - d.window + 1) : 0;
  const int j_first = lo / KRK_PAGE, j_last = pos / KRK_PAGE;
  const int n_pages = j_last - j_first + 1;
  const int per = (n_pages + splits - 1) / splits;
  const int j_lo = j_first + split * per, j_hi = min(j_last, j_lo + per - 1);
  const bool owns_new = j_lo <= j_last && j_last <= j_hi;
  const size_t page_stride = (size_t)a.HKV * KRK_PAGE * D;
  const size_t head_off = (size_t)kh * KRK_PAGE * D;
  const int row_w = (a.HQ + 2 * a.HKV) * D;

  // the new token's rows of this kv head: G query rows, the key row, the value row -> shared memory
  const bf16* qkv_row = a.qkv + (size_t)seq * row_w;
  for (int i = threadIdx.x; i < (G + 2) * (D / 8); i += NTHREADS) {
    const int r = i / (D / 8), c = i % (D / 8);
    const bf16* src = r < G ? qkv_row + (size_t)(kh * G + r) * D : qkv_row + (size_t)(a.HQ + (r - G) * a.HKV + kh) * D;
    *reinterpret_cast<uint4*>(as.rows + (size_t)r * D + c * 8) = __ldcg(reinterpret_cast<const uint4*>(src + c * 8));
  }
  __syncthreads();
  if (worker) {
    const bf16* cos_row = a.cos_t ? a.cos_t + (size_t)pos * (D / 2) : nullptr;
    const bf16* sin_row = a.sin_t ? a.sin_t + (size_t)pos * (D / 2) : nullptr;
    for (int r = warp; r < 16; r += 4) {
      if (r < G) {
        HeadRow row;
        row.load_values(as.rows + (size_t)r * D, d.g_q, d.gains_f32, lane);
        row.load_angles(cos_row, sin_row, lane);
        row.finish(as.q_s + r * DP, d.g_q != nullptr, a.cos_t != nullptr, d.eps_qk, lane);
      } else {
        for (int i = lane; i < D; i += 32) as.q_s[r * DP + i] = __float2bfloat16_rn(0.f);
      }
    }
    if (owns_new && warp == G % 4) {
      HeadRow row;
      row.load_values(as.rows + (size_t)G * D, d.g_k, d.gains_f32, lane);
      row.load_angles(cos_row, sin_row, lane);
      row.finish(as.kv_new, d.g_k != nullptr, a.cos_t != nullptr, d.eps_qk, lane);
      for (int i = lane; i < D; i += 32) as.kv_new[D + i] = as.rows[(size_t)(G + 1) * D + i];
      __syncwarp();
      const int page = d.table[(size_t)slot * d.width + j_last % d.width];
      const size_t at = (size_t)page * page_stride + head_off + (size_t)(pos % KRK_PAGE) * D;
      for (int i = lane; i < D; i += 32) {
        d.k_cache[at + i] = as.kv_new[i];
        d.v_cache[at + i] = as.kv_new[D + i];
      }
    }
  }
  __syncthreads();

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[DTILES][4];
#pragma unroll
  for (int n = 0; n < DTILES; ++n)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[n][c] = 0.f;
  uint32_t qf[KSTEPS][4];
  if (worker) load_q(qf, as.q_s + g * DP, as.q_s + (g + 8) * DP, lane);

  bf16* ks = as.page;
  bf16* vs = as.page + TILE_ELEMS;
  for (int j = j_lo; j <= j_hi; ++j) {
    if (worker) {
      // the page of one kv head is contiguous: all of its pieces are requested, then stored
      const int page = d.table[(size_t)slot * d.width + j % d.width];
      const bf16* ksrc = d.k_cache + (size_t)page * page_stride + head_off;
      const bf16* vsrc = d.v_cache + (size_t)page * page_stride + head_off;
      uint4 kreg[PIECES_PER_THREAD], vreg[PIECES_PER_THREAD];
#pragma unroll
      for (int i = 0; i < PIECES_PER_THREAD; ++i) {
        const int p = threadIdx.x + i * ATT_THREADS;
        if (p < PAGE_PIECES) {
          kreg[i] = __ldcg(reinterpret_cast<const uint4*>(ksrc) + p);
          vreg[i] = __ldcg(reinterpret_cast<const uint4*>(vsrc) + p);
        }
      }
#pragma unroll
      for (int i = 0; i < PIECES_PER_THREAD; ++i) {
        const int p = threadIdx.x + i * ATT_THREADS;
        if (p < PAGE_PIECES) {
          const int key = p / (D / 8), ch = p % (D / 8);
          *reinterpret_cast<uint4*>(ks + kv_off(key, ch)) = kreg[i];
          *reinterpret_cast<uint4*>(vs + kv_off(key, ch)) = vreg[i];
        }
      }
    }
    __syncthreads();
    if (j == j_last) {  // the row of the new token, whether or not the global write has landed
      for (int i = threadIdx.x; i < D; i += NTHREADS) {
        ks[kv_off(pos % KRK_PAGE, i >> 3) + (i & 7)] = as.kv_new[i];
        vs[kv_off(pos % KRK_PAGE, i >> 3) + (i & 7)] = as.kv_new[D + i];
      }
      __syncthreads();
    }
    if (worker) {
      const int key0 = warp * 16;
      float s[2][4];
      qk_tile<2>(s, qf, ks, key0, lane);
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int key = j * KRK_PAGE + key0 + n * 8 + 2 * t4 + (c & 1);
          s[n][c] = (key <= pos && key >= lo) ? s[n][c] * a.scale_log2 : -INFINITY;
        }
      softmax_update<2>(s, m, l, o);
      pv_tile<2>(o, s, vs, key0, lane);
    }
    __syncthreads();
  }

  // the four warps' results, merged in warp order, are this split's partial (m, l, o[D]) per query row
  float* red = reinterpret_cast<float*>(as.page);  // [4][16][RP]
  if (worker) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float* dst = red + ((size_t)warp * 16 + g + 8 * h) * RP;
      if (t4 == 0) { dst[D] = m[h]; dst[D + 1] = l[h]; }
#pragma unroll
      for (int n = 0; n < DTILES; ++n) {
        dst[n * 8 + 2 * t4] = o[n][2 * h];
        dst[n * 8 + 2 * t4 + 1] = o[n][2 * h + 1];
      }
    }
  }
  __syncthreads();
  float* mine = a.att_part + (size_t)item * 16 * RP;
  for (int r = warp; r < G; r += WARPS) {
    float mw[4], big = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) { mw[w] = red[((size_t)w * 16 + r) * RP + D]; big = fmaxf(big, mw[w]); }
    const float safe = big == -INFINITY ? 0.f : big;
    float wgt[4], lsum = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) { wgt[w] = exp2f(mw[w] - safe); lsum += wgt[w] * red[((size_t)w * 16 + r) * RP + D + 1]; }
    for (int i = lane; i < D; i += 32) {
      float acc = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) acc += wgt[w] * red[((size_t)w * 16 + r) * RP + i];
      __stcg(mine + (size_t)r * RP + i, acc);
    }
    if (lane == 0) { __stcg(mine + (size_t)r * RP + D, big); __stcg(mine + (size_t)r * RP + D + 1, lsum); }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(a.att_flags + seq * a.HKV + kh, 1);
    if (old == splits - 1) { __threadfence(); a.att_flags[seq * a.HKV + kh] = 0; }
    word[1] = old;
  }
  __syncthreads();
  if (word[1] == splits - 1) {
    // every split of this (sequence, kv head) has left its partial: merge them in split order
    const float* first = a.att_part + (size_t)(item - split) * 16 * RP;
    for (int r = warp; r < G; r += WARPS) {
      float big = -INFINITY;
      for (int s2 = 0; s2 < splits; ++s2) big = fmaxf(big, __ldcg(first + ((size_t)s2 * 16 + r) * RP + D));
      float lsum = 0.f;
      float acc[(D + 31) / 32];
#pragma unroll
      for (int i = 0; i < (D + 31) / 32; ++i) acc[i] = 0.f;
      for (int s2 = 0; s2 < splits; ++s2) {
        const float* p = first + ((size_t)s2 * 16 + r) * RP;
        const float w = exp2f(__ldcg(p + D) - big);
        lsum += w * __ldcg(p + D + 1);
#pragma unroll
        for (int i = 0; i < (D + 31) / 32; ++i) {
          const int dd = lane + 32 * i;
          if (dd < D) acc[i] += w * __ldcg(p + dd);
        }
      }
      const float inv = 1.0f / lsum;
      bf16* dst = a.attn + ((size_t)seq * a.HQ + kh * G + r) * D;
#pragma unroll
      for (int i = 0; i < (D + 31) / 32; ++i) {
        const int dd = lane + 32 * i;
        if (dd < D) dst[dd] = __float2bfloat16_rn(acc[i] * inv);
      }
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(NTHREADS, 1) decode_layers_kernel(const Args a, int pitch, size_t xs_bytes) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Shared sh;
  sh.ring = reinterpret_cast<uint4*>(smem_raw);
  constexpr size_t RING_BYTES = (size_t)RING * 2 * NTHREADS * 16;
  constexpr size_t RED_BYTES = (size_t)2 * WARPS * 2 * 128 * sizeof(float);
  sh.red = reinterpret_cast<float*>(smem_raw + RING_BYTES);
  sh.word = reinterpret_cast<int*>(smem_raw + RING_BYTES + RED_BYTES);
  sh.xs = reinterpret_cast<bf16*>(smem_raw + RING_BYTES + RED_BYTES + 64);
  AttShared as;
  as.page = sh.xs;
  as.q_s = as.page + 2 * TILE_ELEMS;
  as.kv_new = as.q_s + 16 * DP;
  as.rows = as.kv_new + 2 * D;
  (void)xs_bytes;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gq = lane >> 2, t = lane & 3;

  // the copy side starts at once: RING chunk steps in flight before anything else
  Walk iss, con;
  iss.layer = 0;
  iss.phase = 0;
  iss.enter(a, warp);
  for (int i = 0; i < RING; ++i) {
    if (!iss.done) {
      uint4* dst = sh.ring + (size_t)i * 2 * NTHREADS + threadIdx.x;
      const bf16* src = iss.source(gq, t);
      cp_async_16(dst, src);
      cp_async_16(dst + NTHREADS, src + (size_t)8 * iss.g.K);
      iss.step();
      if (iss.L >= iss.g.end) { iss.next_phase(); iss.enter(a, warp); }
    }
    cp_async_commit();
  }
  unsigned int n_steps = 0, generation = 0;
  int red_buf = 0;
  bf16* x_cur = a.x0;
  bf16* x_other = a.x1;
  bool alive = true;

  for (int layer = 0; layer < a.n_layers && alive; ++layer) {
    const Layer& d = a.layers[layer];
    // 1: norm, qkv
    norm_rows(a, sh, x_cur, layer > 0 ? a.branch : nullptr, layer > 0 ? x_other : nullptr, d.g_attn, d.gains_f32, d.eps_attn, pitch);
    if (layer > 0) { bf16* tmp = x_cur; x_cur = x_other; x_other = tmp; }
    project<true, false>(a, sh, con, iss, n_steps, red_buf, nullptr, a.qkv, pitch, layer, QKV);
    if (!(alive = grid_barrier(a, generation, sh.word))) break;
    // 2: attention
    for (int item = blockIdx.x; item < a.M * a.HKV * a.splits; item += gridDim.x) attention_item(a, d, as, sh.word, item);
    if (!(alive = grid_barrier(a, generation, sh.word))) break;
    // 3: output projection
    project<false, false>(a, sh, con, iss, n_steps, red_buf, a.attn, a.branch, pitch, layer, OUT);
    if (!(alive = grid_barrier(a, generation, sh.word))) break;
    // 4: norm, gate/up, swiglu
    norm_rows(a, sh, x_cur, a.branch, x_other, d.g_mlp, d.gains_f32, d.eps_mlp, pitch);
    { bf16* tmp = x_cur; x_cur = x_other; x_other = tmp; }
    project<true, true>(a, sh, con, iss, n_steps, red_buf, nullptr, a.act, pitch, layer, GATE_UP);
    if (!(alive = grid_barrier(a, generation, sh.word))) break;
    // 5: down projection
    project<false, false>(a, sh, con, iss, n_steps, red_buf, a.act, a.branch, pitch, layer, DOWN);
    if (!(alive = grid_barrier(a, generation, sh.word))) break;
  }
  cp_async_wait<0>();
}

}  // namespace decode_layers
