// Paged prefill attention on the fifth-generation tensor cores (tcgen05), bfloat16: rows that
// bring more than one token (portions of prompts), causal, over the block table.
//
// A block owns 128 queries of one head; keys and values of the row's pages come in tiles of
// 128 keys.  Both products run as tcgen05.mma with the accumulators in tensor memory (TMEM):
//
//   S = Q K^T      A = Q [128 x hd] and B = K [128 keys x hd] from shared memory, both
//                  K-major; S[128 x 128] float in TMEM
//   O += P V       A = P [128 x 128 keys] bfloat16 from shared memory, where the softmax threads
//                  write it in the swizzled layout a TMA load would leave; B = V [128 keys x hd]
//                  from shared memory exactly as it lies in the cache (hd contiguous), read
//                  "MN-major"; O[128 x hd] float stays in TMEM
//
// Tiles alternate between two halves of the block that do not wait for each other.  Half w
// (softmax warps 4w..4w+3, score buffer S_w, accumulator O_w, P buffer P_w) takes tiles w,
// w + 2, ...; it keeps a running maximum and sum of its own, and the two accumulators are merged
// at the end like the partial results of a split softmax.  So while one half exponentiates, the
// other reads its scores or waits for them, and the tensor cores always have a product to do.
//
//   warps 0-7   softmax: thread r of a half owns query r, which is lane r of the TMEM, so a
//               row's maximum and sum need no exchange between threads.  The row comes into
//               registers in one round trip, and the score buffer is released at once, so that
//               the scores of the half's next tile are computed while these are exponentiated.
//               O_w is rescaled in TMEM only when the row maximum grew by more than 2^8 since it
//               was last fixed (below that the old maximum stays in use, which changes nothing
//               but the common factor of P and the sum).
//   warps 8, 9  producers, one for K and one for V: they look the tile's pages up in the block
//               table.  Pages that follow one another in the pool come as one TMA box per half
//               of the head (a 4-D view of the cache: a run of pages of one head); otherwise
//               one box [page x 64] per page and half, which costs the warp some 75 cycles a box.
//   warp 10     issues the score products: S(0), S(1), then S(j + 2) when S(j) is in registers
//   warp 11     issues P(j) V(j) when P(j) is written
//
// The queries' own keys were appended before this kernel runs, so a portion of a prompt
// attends to the cache and to itself alike.  Pages past a row's last one are replaced by the
// tile's first page: their scores are masked, and what is multiplied by the zeros is then
// finite.  Every wait is bounded; when one gives up the block records it, stores nothing,
// frees its tensor memory and returns.
#include "common.cuh"
#include "attention_params.h"
#include "tcgen05_helpers.cuh"
#include <cstdlib>

namespace {
constexpr int QT = 128;            // queries per block (rows of both MMAs)
constexpr int KT = 128;            // keys per tile
constexpr int HALF_THREADS = 128;  // softmax threads of one half
constexpr int PRODUCER_WARP0 = 8, MMA_WARP = 10;   // warp 10 issues the score products, warp 11 the P V products
constexpr int THREADS = (MMA_WARP + 2) * 32;
constexpr int BOX_BYTES = 128 * 128;   // 128 rows of one 128-byte swizzle row each
constexpr float RESCALE_STEP = 8.f;    // in powers of two
constexpr int TMEM_COLS = 512;
constexpr int COL_S = 0, COL_O = 2 * KT;   // S_0, S_1, then O_0, O_1

template <int HD>
struct Layout {
  static constexpr int HALVES = HD / 64;
  static constexpr int STAGES = 2;    // two, because a stage is freed by the barrier of the tile two before (see the producers)
  static constexpr int Q_BYTES = HALVES * BOX_BYTES;
  static constexpr int TILE_BYTES = HALVES * BOX_BYTES;   // one K or V tile
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + STAGES * TILE_BYTES;
  static constexpr int OFF_P = OFF_V + STAGES * TILE_BYTES;           // P of each half: two boxes [128 x 64 keys]
  static constexpr int P_BYTES = 2 * BOX_BYTES;
  static constexpr int TOTAL = OFF_P + 2 * P_BYTES + 1024;            // 1024 to start on a swizzle boundary
};

// 2^x by the special-function unit (two units in the last place; results below 2^-126 become 0)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// One piece of work: 128 queries of one head of one row.  Pieces are numbered with the head fastest, then the rows,
// then the query tiles of each row from its latest (which has the most keys) to its first: from long to short.
struct Piece {
  int row, h, qt, nq, t0, pos0, last_pos, kt_first, n_tiles, last_page;
  bool valid;
};

__device__ __forceinline__ Piece piece_of(const DkAttnParams& p, int index, int row_lo, int n_rows) {
  Piece w;
  w.h = index % p.H;
  w.row = row_lo + (index / p.H) % n_rows;
  const int yy = index / (p.H * n_rows);                // 0: the row's latest query tile, which has the most keys
  const int q_len = p.row_q_len[w.row];
  w.qt = (q_len + QT - 1) / QT - 1 - yy;
  const int q0 = w.qt * QT;
  w.valid = !(p.row_filter == 2 && q_len == 1) && w.qt >= 0;
  w.nq = min(QT, q_len - q0);
  w.t0 = p.row_q_start[w.row] + q0;
  w.pos0 = p.row_pos_start[w.row] + q0;
  w.last_pos = w.pos0 + w.nq - 1;
  const int lo = (p.window > 0 && w.pos0 - p.window + 1 > 0) ? w.pos0 - p.window + 1 : 0;
  w.kt_first = lo / KT;
  w.n_tiles = w.valid ? w.last_pos / KT - w.kt_first + 1 : 0;
  w.last_page = w.last_pos / p.ps;
  return w;
}

// A block takes several pieces, one after the other.  With as many blocks as SMs
// the barriers, the tensor memory and the descriptors are set up once per SM instead of once per piece, and the next
// piece's queries, first keys and first scores are asked for and computed while the softmax threads still merge and
// write the piece before.  Every barrier is used by the tiles of one parity (tile j of a piece by the barriers of
// class j % 2, as is its stage of K and V), so what a wait needs is the number of tiles of that class the block
// has had so far: `had[c]`, counted alike by every warp.
template <int HD>
__global__ void __launch_bounds__(THREADS, 1) attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                          const __grid_constant__ CUtensorMap map_kv,
                                                                          const __grid_constant__ CUtensorMap map_run,
                                                                          const DkAttnParams p, const int n_qt) {
  using L = Layout<HD>;
  constexpr int STAGES = L::STAGES;
  static_assert(STAGES == 2, "a stage belongs to the tiles of one parity");

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  // barriers: q_full, k_full[2], v_full[2], s_full[2], p_full[2], o_done[2], merge, s_free[2], piece_done
  __shared__ __align__(8) unsigned long long bars[1 + 2 + 2 + 2 + 2 + 2 + 1 + 2 + 1];
  // row_stat(w)[query]: maximum and sum of half w's tiles, for the merge; it lies over the half's P, which
  // is no longer read when the half has seen its last product complete
  auto row_stat = [&](int w) { return reinterpret_cast<float2*>(smem + L::OFF_P + w * L::P_BYTES); };
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int failed;
  __shared__ int row_range[2];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ps = p.ps, G = p.H / p.KV;

  const uint32_t bar0 = s2u(&bars[0]);
  const uint32_t q_full = bar0;
  const uint32_t k_full = bar0 + 8, v_full = k_full + 16, s_full = v_full + 16, p_full = s_full + 16, o_done = p_full + 16,
                 merge_bar = o_done + 16, s_free = merge_bar + 8, piece_done = s_free + 16;
  if (tid == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(k_full + 8 * s, 1);
      mbar_init(v_full + 8 * s, 1);
    }
    for (int w = 0; w < 2; ++w) {
      mbar_init(s_full + 8 * w, 1);
      mbar_init(p_full + 8 * w, HALF_THREADS);
      mbar_init(o_done + 8 * w, 1);
      mbar_init(s_free + 8 * w, HALF_THREADS);
    }
    mbar_init(merge_bar, 2 * HALF_THREADS);
    mbar_init(piece_done, 2 * HALF_THREADS);
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    // In a step that also holds single tokens (which the decode kernel takes) only the rows from the first to the
    // last one that brings several tokens are cut into pieces: a block does not have to walk over hundreds of rows
    // that are not its business.
    int lo = p.rows, hi = -1;
    if (p.row_filter == 2) {
      for (int r0 = 0; r0 < p.rows; r0 += 32) {
        const int r = r0 + lane;
        if (r < p.rows && p.row_q_len[r] > 1) {
          lo = min(lo, r);
          hi = max(hi, r);
        }
      }
      lo = __reduce_min_sync(0xffffffffu, lo);
      hi = __reduce_max_sync(0xffffffffu, hi);
    } else {
      lo = 0;
      hi = p.rows - 1;
    }
    if (lane == 0) {
      row_range[0] = lo;
      row_range[1] = hi;
    }
  }
  if (warp == MMA_WARP) tmem_alloc(s2u(&tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const int row_lo = row_range[0], n_rows = max(0, row_range[1] - row_range[0] + 1);
  const int n_pieces = p.H * n_qt * n_rows;
  // The pieces a block takes: in rounds of gridDim.x pieces, forwards in the even rounds and backwards in the odd ones.
  // Pieces are numbered from long to short, so a block that got a long one in one round gets a short one in the next,
  // and all blocks end at about the same time without asking each other anything.
  auto piece_index = [&](int round) {
    const int b = (round & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x;
    return round * (int)gridDim.x + b;
  };
  const uint32_t tmem = tmem_slot;
  const uint32_t sm_q = s2u(smem + L::OFF_Q), sm_k = s2u(smem + L::OFF_K), sm_v = s2u(smem + L::OFF_V),
                 sm_p = s2u(smem + L::OFF_P);
  int had0 = 0, had1 = 0;   // tiles of each parity in the pieces before the current one (scalars: an array indexed by a
                            // value the compiler does not know would live in local memory)
  int n_done = 0;           // pieces before the current one

  // The four warps that fetch and issue need few registers, the eight softmax warps hold a row of 128 scores each:
  // the first warpgroup gives registers back and the other two take them (384 threads x 168 = 128 x 64 + 256 x 216).
  // (Each change of the register count stands inside the branch whose code it is for: after a common point the
  // compiler would have to assume the smaller count for everybody.)
  if (warp >= PRODUCER_WARP0) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 64;\n");
  if (warp < MMA_WARP) {      // (the three branches of this warpgroup keep their indentation)
    // ----------------------------------------------------------- producers
    // one warp for K and one for V, so that the next K is never held up behind a V whose buffer
    // is still being read
    const int kind = warp - PRODUCER_WARP0;     // 0: K, 1: V
    const int ppt = KT / ps;      // pages per tile, at most 16
    // A stage of K is free when the scores made from it are complete, a stage of V when the product
    // with it is: the producers wait on the same barriers as the softmax threads.
    const uint32_t full = kind ? v_full : k_full, done = kind ? o_done : s_full, sm_dst = kind ? sm_v : sm_k;
    int q_asked = 0;
    int asked0 = 0, asked1 = 0;   // tiles of each parity asked for so far
    for (int round = 0; round * (int)gridDim.x < n_pieces && !failed; ++round) {
      const int index = piece_index(round);
      if (index >= n_pieces) continue;
      const Piece w = piece_of(p, index, row_lo, n_rows);
      if (!w.valid) continue;
      const int kvh = w.h / G;
      if (kind == 0) {
        // the queries' buffer is free when every score product of the piece before is complete
        bool ok = true;
        if (n_done > 0) ok = mbar_wait(s_full, (had0 - 1) & 1) && mbar_wait(s_full + 8, (had1 - 1) & 1);
        if (!__all_sync(0xffffffffu, ok && !failed)) { failed = 1; break; }
        if (lane == 0) {
          mbar_expect_tx(q_full, (uint32_t)L::Q_BYTES);
          for (int half = 0; half < L::HALVES; ++half)
            tma_load_2d(sm_q + half * BOX_BYTES, &map_q, w.h * HD + half * 64, w.t0, q_full);   // rows past the last token are zeros
        }
        q_asked = n_done + 1;
      }
      for (int j = 0; j < w.n_tiles; ++j) {
        const int c = j & 1, ord = (c ? had1 : had0) + j / 2;     // the ord-th tile of its parity in this block
        const int lp = (w.kt_first + j) * ppt + lane;
        int page = -1;
        if (lane < ppt && lp <= w.last_page && lp < p.max_pages) {
          page = p.block_table[(size_t)w.row * p.max_pages + lp];
          if (page < 0 || page >= p.num_pages) {
            dk_report(p.err, DK_DEV_BAD_PAGE, w.row, lp, page);
            page = -1;
          }
        }
        int first = __shfl_sync(0xffffffffu, page, 0);
        // a tile whose pages follow one another in the pool comes with one request per half of the head
        const bool run = __all_sync(0xffffffffu, lane >= ppt || (page >= 0 && page == first + lane));
        if (first < 0) first = 0;
        if (page < 0) page = first;
        const int grow = ((page * 2 + kind) * p.KV + kvh) * ps;    // row of the cache seen as [pages * 2 * KV * ps, hd]
        bool ok = true;
        if (ord >= 1) ok = mbar_wait(done + 8 * c, (ord - 1) & 1);
        if (!__all_sync(0xffffffffu, ok && !failed)) { failed = 1; break; }
        if (lane == 0) mbar_expect_tx(full + 8 * c, (uint32_t)L::TILE_BYTES);
        __syncwarp();
        if (run) {
          if (lane == 0)
            for (int half = 0; half < L::HALVES; ++half)
              tma_load_4d(sm_dst + c * L::TILE_BYTES + half * BOX_BYTES, &map_run, half * 64, 0, kind * p.KV + kvh, first, full + 8 * c);
        } else if (lane < ppt) {
          for (int half = 0; half < L::HALVES; ++half)
            tma_load_2d(sm_dst + c * L::TILE_BYTES + half * BOX_BYTES + lane * ps * 128, &map_kv, half * 64, grow, full + 8 * c);
        }
        if (c) asked1 = ord + 1; else asked0 = ord + 1;
      }
      if (failed) break;
      had0 += (w.n_tiles + 1) / 2;
      had1 += w.n_tiles / 2;
      ++n_done;
    }
    if (failed && lane == 0) {
      // nobody may leave while copies of this block are in flight: wait (bounded) for the last ones asked for
      if (kind == 0 && q_asked > 0) mbar_wait(q_full, (q_asked - 1) & 1);
      if (asked0 > 0) mbar_wait(full, (asked0 - 1) & 1);
      if (asked1 > 0) mbar_wait(full + 8, (asked1 - 1) & 1);
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------- MMA issuer of the scores
    // The whole warp runs the loop, so that descriptors and addresses stay warp-uniform; one
    // elected lane issues.  The scores of a tile are computed as soon as its keys have arrived and the
    // softmax threads hold the scores of the tile of the same parity before it in registers.
    const bool leader = elect_one();
    const uint32_t idesc_s = instr_desc_bf16(QT, KT, false);
    auto wait_all = [&](uint32_t bar, uint32_t parity) -> bool {     // the same answer in every lane
      return __all_sync(0xffffffffu, mbar_wait(bar, parity));
    };
    const uint64_t da0 = smem_desc_k_major(sm_q);
    bool ok = true;
    for (int round = 0; ok && round * (int)gridDim.x < n_pieces; ++round) {
      const int index = piece_index(round);
      if (index >= n_pieces) continue;
      const Piece w = piece_of(p, index, row_lo, n_rows);
      if (!w.valid) continue;
      ok = wait_all(q_full, n_done & 1);
      for (int j = 0; ok && j < w.n_tiles; ++j) {
        const int c = j & 1, ord = (c ? had1 : had0) + j / 2;
        if (ord >= 1 && !wait_all(s_free + 8 * c, (ord - 1) & 1)) { ok = false; break; }
        if (!wait_all(k_full + 8 * c, ord & 1)) { ok = false; break; }
        tc_fence_after();
        const uint64_t db0 = smem_desc_k_major(sm_k + c * L::TILE_BYTES);
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            const uint64_t off = (uint64_t)(((kk / 4) * BOX_BYTES + (kk % 4) * 32) >> 4);   // start addresses count 16 bytes
            umma(tmem + COL_S + c * KT, da0 + off, db0 + off, idesc_s, kk > 0 ? 1u : 0u);
          }
          umma_commit(s_full + 8 * c);
        }
        __syncwarp();
      }
      had0 += (w.n_tiles + 1) / 2;
      had1 += w.n_tiles / 2;
      ++n_done;
    }
    if (!ok) failed = 1;
  } else if (warp == MMA_WARP + 1) {
    // ------------------------------------------ MMA issuer of P V
    const bool leader = elect_one();
    const uint32_t idesc_o = instr_desc_bf16(QT, HD, true);
    auto wait_all = [&](uint32_t bar, uint32_t parity) -> bool {
      return __all_sync(0xffffffffu, mbar_wait(bar, parity));
    };
    bool ok = true;
    for (int round = 0; ok && round * (int)gridDim.x < n_pieces; ++round) {
      const int index = piece_index(round);
      if (index >= n_pieces) continue;
      const Piece w = piece_of(p, index, row_lo, n_rows);
      if (!w.valid) continue;
      for (int j = 0; ok && j < w.n_tiles; ++j) {
        const int c = j & 1, ord = (c ? had1 : had0) + j / 2;
        if (!wait_all(v_full + 8 * c, ord & 1) || !wait_all(p_full + 8 * c, ord & 1)) { ok = false; break; }
        tc_fence_after();
        const uint64_t dp0 = smem_desc_k_major(sm_p + c * L::P_BYTES);
        const uint64_t dv0 = smem_desc_mn_major(sm_v + c * L::TILE_BYTES, BOX_BYTES);
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < KT / 16; ++kk)   // 16 keys further: 32 bytes along a row of P, two groups of 8 rows of V
            umma(tmem + COL_O + c * HD, dp0 + (uint64_t)(((kk / 4) * BOX_BYTES + (kk % 4) * 32) >> 4),
                 dv0 + (uint64_t)(kk * (2048 >> 4)), idesc_o, (j > 1 || kk > 0) ? 1u : 0u);
          umma_commit(o_done + 8 * c);
        }
        __syncwarp();
      }
      had0 += (w.n_tiles + 1) / 2;
      had1 += w.n_tiles / 2;
      ++n_done;
    }
    if (!ok) failed = 1;
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;\n");
    // ------------------------------------------------------------- softmax
    const int w = warp >> 2;                            // which half: its tiles are w, w + 2, ...
    const int r = (warp & 3) * 32 + lane;               // query of this thread = lane of the TMEM
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem + lane_base + COL_S + w * KT;    // scores of this half
    const uint32_t t_o = tmem + lane_base + COL_O + w * HD;
    const float sl2 = p.scale * 1.4426950408889634f;
    const int window = p.window;
    bool good = true;
    int had_w = 0;            // tiles of this half in the pieces before the current one
#pragma unroll 1
    for (int round = 0; good && round * (int)gridDim.x < n_pieces; ++round) {
      const int index = piece_index(round);
      if (index >= n_pieces) continue;
      const Piece pc = piece_of(p, index, row_lo, n_rows);
      if (!pc.valid) continue;
      const int n_tiles = pc.n_tiles, pos0 = pc.pos0, last_pos = pc.last_pos, kt_first = pc.kt_first, nq = pc.nq, t0 = pc.t0, h = pc.h;
      const int qpos = pos0 + r;
      float m_used = -INFINITY, l_sum = 0.f;
      int mine = 0;                                       // tiles of this half in this piece so far
      // Before this half writes a P again (which lies where its maximum and sum for the merge lay) and lets the
      // P V product overwrite an accumulator, both halves must have finished reading them for the piece before.
      if (n_done > 0) {
        bool ok = mbar_wait(piece_done, (n_done - 1) & 1);
        if (!__all_sync(0xffffffffu, ok && !failed)) { failed = 1; good = false; break; }
      }
      for (int j = w; j < n_tiles; j += 2, ++mine) {
        const int ord = had_w + mine;
        bool ok = mbar_wait(s_full + 8 * w, ord & 1);
        if (!__all_sync(0xffffffffu, ok && !failed)) { failed = 1; good = false; break; }
        tc_fence_after();
        const int kbase = (kt_first + j) * KT;
        const bool edge = (kbase + KT - 1 > pos0) || (window > 0 && kbase < last_pos - window + 1);
        // the whole row comes into registers in one round trip; the score buffer is free for the
        // scores of this half's next tile at once
        float v[KT];
#pragma unroll
        for (int c = 0; c < KT / 32; ++c) tmem_ld32_nowait(t_s + c * 32, v + c * 32);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(s_free + 8 * w);
        if (edge) {
          const int hi = qpos - kbase, lo = window > 0 ? qpos - window - kbase : -1;
#pragma unroll
          for (int i = 0; i < KT; ++i)     // key kbase + i is seen by query qpos when it is not later and not before the window
            if (!(i <= hi && i > lo)) v[i] = -INFINITY;
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains instead of one long one
#pragma unroll
        for (int i = 0; i < KT; i += 4) {
          mx4[0] = fmaxf(mx4[0], v[i]);
          mx4[1] = fmaxf(mx4[1], v[i + 1]);
          mx4[2] = fmaxf(mx4[2], v[i + 2]);
          mx4[3] = fmaxf(mx4[3], v[i + 3]);
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        const float m_new = fmaxf(m_used, mx * sl2);
        const bool grow = m_new > m_used + RESCALE_STEP;      // also the first finite maximum of a row
        float factor = 1.f;
        if (grow) {
          factor = m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_new);
          m_used = m_new;
        }
        const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
        if (mine > 0) {
          // P V of this half's tile before is done: its P may be overwritten, and O_w is at rest
          ok = mbar_wait(o_done + 8 * w, (ord - 1) & 1);
          if (!__all_sync(0xffffffffu, ok && !failed)) { failed = 1; good = false; break; }
          if (__any_sync(0xffffffffu, grow)) {
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
              float o[32];
              tmem_ld32_nowait(t_o + c * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] *= factor;
              tmem_st32(t_o + c * 32, o);
            }
            tmem_wait_st();
            tc_fence_before();
          }
        }
        // exponentials, their sum, and P as bfloat16 in the layout a TMA load with 128-byte swizzle
        // would leave: two boxes of 64 keys, rows of 128 bytes, 16-byte chunks exchanged by the row
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        const uint32_t p_row = sm_p + w * L::P_BYTES + r * 128;
#pragma unroll
        for (int c = 0; c < KT / 8; ++c) {
          float e[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            e[i] = fast_exp2(fmaf(v[c * 8 + i], sl2, neg_m));
            sum4[i & 3] += e[i];
          }
          const uint32_t addr = p_row + (c / 8) * BOX_BYTES + (((c % 8) ^ (r & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(addr), "r"(pack2(e[0], e[1])), "r"(pack2(e[2], e[3])),
                       "r"(pack2(e[4], e[5])), "r"(pack2(e[6], e[7])) : "memory");
        }
        l_sum = l_sum * factor + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        fence_async_smem();
        mbar_arrive(p_full + 8 * w);
      }
      if (good && mine > 0) {
        bool ok = mbar_wait(o_done + 8 * w, (had_w + mine - 1) & 1);
        if (!__all_sync(0xffffffffu, ok && !failed)) { failed = 1; good = false; }
      }
      // merge of the two halves: each tells the other its maximum and sum, then writes half of the columns
      row_stat(w)[r] = make_float2(m_used, l_sum);
      tc_fence_before();
      mbar_arrive(merge_bar);
      if (good) {
        bool ok = mbar_wait(merge_bar, n_done & 1);
        if (!__all_sync(0xffffffffu, ok && !failed)) { failed = 1; good = false; }
      }
      if (good) {
        tc_fence_after();
        const float2 other = row_stat(w ^ 1)[r];
        const float m_all = fmaxf(m_used, other.x);
        const float f_mine = m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_all);
        const float f_other = other.x == -INFINITY ? 0.f : fast_exp2(other.x - m_all);
        const float l_all = l_sum * f_mine + other.y * f_other;
        const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
        const float f0 = (w == 0 ? f_mine : f_other) * inv, f1 = (w == 0 ? f_other : f_mine) * inv;
        const bool two = n_tiles > 1;                     // O_1 holds nothing when there was one tile
        constexpr int OC = HD / 64;                       // chunks of 32 columns this thread writes
        __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + ((size_t)(t0 + r) * p.H + h) * HD + w * (HD / 2);
#pragma unroll
        for (int c = 0; c < OC; ++c) {
          float o0[32], o1[32];
          const uint32_t col = (uint32_t)(w * (HD / 2) + c * 32);
          tmem_ld32_nowait(tmem + lane_base + COL_O + col, o0);
          if (two) tmem_ld32_nowait(tmem + lane_base + COL_O + HD + col, o1);
          tmem_wait_ld();
          if (c == OC - 1) {
            // the accumulators and the other half's maximum and sum are in registers: the next piece may overwrite them
            tc_fence_before();
            mbar_arrive(piece_done);
          }
          if (r < nq) {
#pragma unroll
            for (int i = 0; i < 32; ++i) o0[i] = two ? o0[i] * f0 + o1[i] * f1 : o0[i] * f0;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 st;
              st.x = pack2(o0[v * 8], o0[v * 8 + 1]);
              st.y = pack2(o0[v * 8 + 2], o0[v * 8 + 3]);
              st.z = pack2(o0[v * 8 + 4], o0[v * 8 + 5]);
              st.w = pack2(o0[v * 8 + 6], o0[v * 8 + 7]);
              *reinterpret_cast<uint4*>(orow + c * 32 + v * 8) = st;
            }
          }
        }
        if (p.lse != nullptr && r < nq && w == 0)
          p.lse[(size_t)(t0 + r) * p.H + h] = l_all > 0.f ? m_all * 0.6931471805599453f + logf(l_all) : -INFINITY;
      }
      had_w += (n_tiles + 1 - w) / 2;
      ++n_done;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (failed && tid == 0) dk_report(p.err, DK_DEV_TIMEOUT, (int)blockIdx.x, (int)gridDim.x, n_pieces);
  if (warp == MMA_WARP) tmem_dealloc(tmem, TMEM_COLS);
}

template <int HD>
int launch(const DkAttnParams& p, int max_q_len, cudaStream_t stream) {
  using L = Layout<HD>;
  CUtensorMap map_q, map_kv, map_run;
  const long long kv_rows = (long long)p.num_pages * 2 * p.KV * p.ps;
  DK_REQUIRE(kv_rows < (1ll << 31), "attention_prefill_tc: the cache of one layer has too many rows for a tensor map coordinate");
  DK_REQUIRE(make_tensor_map_bf16(&map_q, p.q, p.T, p.H * HD, p.q_stride, QT),
             "attention_prefill_tc: cannot encode the tensor map of the queries");
  DK_REQUIRE(make_tensor_map_bf16(&map_kv, p.kv, kv_rows, HD, HD, p.ps),
             "attention_prefill_tc: cannot encode the tensor map of the cache");
  // the cache as [page][K|V, head][offset][hd]: a run of pages of one head in one box
  const unsigned long long dims[4] = {(unsigned long long)HD, (unsigned long long)p.ps, (unsigned long long)(2 * p.KV),
                                      (unsigned long long)p.num_pages};
  const unsigned long long strides[3] = {(unsigned long long)HD * 2, (unsigned long long)p.ps * HD * 2,
                                         (unsigned long long)2 * p.KV * p.ps * HD * 2};
  DK_REQUIRE(make_tensor_map_bf16_4d(&map_run, p.kv, dims, strides, p.ps, KT / p.ps),
             "attention_prefill_tc: cannot encode the tensor map of runs of pages");
  static bool configured_on[DK_MAX_DEVICES] = {false};
  bool& configured = configured_on[dk_current_device()];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) {
      dk_set_error("attention_prefill_tc: cannot get %d bytes of shared memory: %s", L::TOTAL, cudaGetErrorString(e));
      return DK_ERR_LAUNCH;
    }
    configured = true;
  }
  const int n_qt = (max_q_len + QT - 1) / QT;
  const long long pieces = (long long)p.H * n_qt * p.rows;
  DK_REQUIRE(pieces < (1ll << 30), "attention_prefill_tc: too many pieces of work");
  const int sms = dk_sm_count();
  static const bool one_each = getenv("DELTA_B200_PREFILL_ONE_PIECE_PER_BLOCK") != nullptr;   // for measurements: a block per piece
  const int blocks = (int)(one_each || pieces < sms ? pieces : sms);
  attention_prefill_tc_kernel<HD><<<blocks, THREADS, L::TOTAL, stream>>>(map_q, map_kv, map_run, p, n_qt);
  return dk_check_launch("attention_prefill_tc");
}
}  // namespace

extern "C" int dk_attention_prefill_tc_supported(int dtype, int H, int KV, int hd, int ps, int q_stride) {
  if (dtype != DK_BF16 || KV <= 0 || H % KV != 0) return 0;
  if (hd != 64 && hd != 128) return 0;
  if (ps != 8 && ps != 16 && ps != 32 && ps != 64 && ps != 128) return 0;
  if (q_stride % 8 != 0) return 0;
  return 1;
}

// max_q_len: the most tokens any row brings (sizes the grid).
extern "C" int dk_attention_prefill_tc(const DkAttnParams* pp, int max_q_len, cudaStream_t stream) {
  const DkAttnParams& p = *pp;
  if (p.T == 0 || p.rows == 0) return 0;
  DK_REQUIRE(dk_attention_prefill_tc_supported(p.dtype, p.H, p.KV, p.hd, p.ps, p.q_stride),
             "attention_prefill_tc: sizes not taken (bfloat16, head size 64 or 128, page size 8 to 128 and a power of two, "
             "query stride a multiple of 8): dtype=%d H=%d KV=%d hd=%d ps=%d stride=%d", p.dtype, p.H, p.KV, p.hd, p.ps, p.q_stride);
  DK_REQUIRE(max_q_len >= 1, "attention_prefill_tc: max_q_len must be positive");
  DK_REQUIRE(p.scale > 0.f, "attention_prefill_tc: the scale of the scores must be positive");
  DK_REQUIRE(p.row_q_start && p.row_q_len && p.row_pos_start && p.block_table, "attention_prefill_tc: row tables are missing");
  DK_REQUIRE((max_q_len + QT - 1) / QT <= 65535 && p.rows <= 65535, "attention_prefill_tc: grid too large");
  DK_REQUIRE(((uintptr_t)p.q % 16) == 0 && ((uintptr_t)p.kv % 16) == 0 && ((uintptr_t)p.out % 16) == 0,
             "attention_prefill_tc: queries, cache and output must start on 16-byte boundaries");
  return p.hd == 64 ? launch<64>(p, max_q_len, stream) : launch<128>(p, max_q_len, stream);
}
