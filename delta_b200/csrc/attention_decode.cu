// Paged decode attention for bfloat16: one new token per request, the keys split
// over several thread blocks, the query heads of one key-value head packed as the
// rows of a tensor-core tile.
//
// Grid (splits, kv heads, batch rows); 4 warps per block.  A block walks its share of
// the request's pages in tiles of 64 keys.  K and V tiles come into shared memory
// with cp.async (3 stages), 16-byte chunks swizzled so that ldmatrix reads without
// bank conflicts.  Each warp owns 16 keys of a tile: S = Q K^T with
// mma.sync.m16n8k16 (rows = the G <= 16 query heads of the group), an online softmax
// in float on its own keys, then O += P V.  The four warps are merged through shared
// memory at the end; with more than one split the block writes (m, l, O) to the
// scratch buffer and a second kernel merges the splits in a fixed order.  With two to
// eight splits the blocks of one (row, key-value head) can instead be launched as one
// thread-block cluster: each keeps (m, l, O) in its own shared memory, and after a
// cluster barrier block r merges the r-th share of the output columns from all of them
// over distributed shared memory, in the same order with the same arithmetic, so that
// neither the scratch buffer nor the second kernel is needed.
//
// The kernel is bound by the bytes of K and V it has to read once; the tensor-core
// work is small beside it, which is why the legacy warp-level MMA is enough here.
//
// TMA variant (pages of 8 tokens or more, no score dump): a tile whose pages follow one another
// in the pool and are wholly visible to the query is fetched by one thread with one TMA box per
// half of the head and K/V (a 4-D view of the cache: a run of pages of one head) instead of 16
// cp.async per thread with their address arithmetic, which is a third of the loop's
// instructions.  Tiles at a window's or the request's edge, scattered pages and chosen pages
// keep the cp.async path with its groups; a TMA tile is waited for on its stage's mbarrier.  The shared-memory layout
// of this variant is the one TMA's 128-byte swizzle leaves: halves of the head side by side,
// rows of 128 bytes, 16-byte chunks exchanged by the row's number.
//
// It takes: the whole cache, a window of it, or the list of chosen pages of DELTA's
// subset layers; and it can dump the scaled scores and the log-sum-exp for DELTA's
// page scoring (reference: backend.py:191-221, 562-577).
#include "common.cuh"
#include "attention_params.h"
#include "mma_helpers.cuh"
#include "tcgen05_helpers.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace {
constexpr int TILE = 64;     // keys per tile
constexpr int STAGES = 3;
constexpr int NWARPS = 4;
constexpr int NTHREADS = NWARPS * 32;

struct RowInfo {
  int t, pos, lo, slot, n_entries, first_page;
  bool subset, dumping;
  const int* sel;
};

__device__ __forceinline__ RowInfo row_info(const DkAttnParams& p, int row) {
  RowInfo r;
  // independent loads first: the position follows from the row's start and length, so that
  // nothing here waits for another load except the count of chosen pages
  const int q_start = p.row_q_start[row], q_len = p.row_q_len[row];
  const int pos_start = p.row_pos_start ? p.row_pos_start[row] : -1;
  r.slot = p.row_slot ? p.row_slot[row] : row;
  const int flags = p.row_flags ? p.row_flags[row] : 0;
  r.t = q_start + q_len - 1;
  r.pos = pos_start >= 0 ? pos_start + q_len - 1 : p.tok_pos[r.t];
  int n_sel = -1;
  if (p.sel_pages != nullptr && (flags & 1)) n_sel = p.sel_count[r.slot];
  r.subset = n_sel >= 0;
  r.lo = (p.window > 0 && r.pos - p.window + 1 > 0) ? r.pos - p.window + 1 : 0;
  r.first_page = r.lo / p.ps;
  r.n_entries = r.subset ? n_sel : (r.pos / p.ps - r.first_page + 1);
  r.sel = r.subset ? p.sel_pages + (size_t)r.slot * p.sel_stride : nullptr;
  r.dumping = p.dump != nullptr && (flags & 1);
  return r;
}

// scratch layout per (row, head, split): HD floats of O, then m and l at the end of the buffer
__device__ __forceinline__ size_t part_o_index(const DkAttnParams& p, int row, int h, int split, int HD) {
  return (((size_t)row * p.H + h) * p.splits + split) * HD;
}
__device__ __forceinline__ size_t part_ml_index(const DkAttnParams& p, int row, int h, int split) {
  return (size_t)p.rows * p.H * p.splits * p.hd + (((size_t)row * p.H + h) * p.splits + split) * 2;
}

// LOW: at most 8 query heads per key-value head.  Rows 8..15 of the MMA tile are then empty;
// their accumulators are two dummy registers that stay zero, and the softmax and the output
// keep one row per thread instead of two, which halves that work and frees registers.
template <bool LOW>
__device__ __forceinline__ void mma_rows(float* c, float (&zd)[2], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (LOW) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(zd[0]), "+f"(zd[1])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// Byte offset of 16-byte chunk ``chunk`` of key ``tok`` inside a K or V tile.
template <int HD, bool TMA>
__device__ __forceinline__ uint32_t tile_offset(int tok, int chunk) {
  if constexpr (TMA) return (uint32_t)((chunk >> 3) * (TILE * 128) + tok * 128 + (((chunk & 7) ^ (tok & 7)) << 4));
  else return (uint32_t)(tok * (HD * 2) + ((chunk ^ (tok & 7)) * 16));
}

template <int HD, bool LOW, bool TMA>
__global__ void __launch_bounds__(NTHREADS, 2) attention_decode_kernel(const __grid_constant__ CUtensorMap map_run,
                                                                       const DkAttnParams p) {
  constexpr int R = LOW ? 1 : 2;              // rows of the tile a thread keeps (g, and g + 8)
  constexpr int CHUNKS = HD / 8;              // 16-byte chunks per key row
  constexpr int ROW_BYTES = HD * 2;
  constexpr int TILE_BYTES = TILE * ROW_BYTES;  // one of K or V
  constexpr int KB = HD / 16;                 // k-blocks of the QK product
  constexpr int NT = HD / 8;                  // n-tiles of the PV product
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // the TMA variant needs its tiles on a 1024-byte boundary (the swizzle pattern repeats every 1024 bytes)
  unsigned char* smem = TMA ? reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023) : smem_raw;
  unsigned char* kv_smem = smem;                                  // STAGES * 2 * TILE_BYTES
  int* s_key = reinterpret_cast<int*>(smem + STAGES * 2 * TILE_BYTES);  // STAGES * TILE key positions (-1: no key)
  int* s_lp = s_key + STAGES * TILE;     // logical page of each of this block's entries
  int* s_page = s_lp + p.block_entries;       // its physical page, -1: none (p.block_entries = entries a block can have)
  int* s_run = s_page + p.block_entries;      // TMA: first physical page of a tile that is one visible run of pages, else -1
  __shared__ __align__(8) unsigned long long full_bar[STAGES];   // TMA: a stage's tile has arrived
  __shared__ int s_timeout;                                       // TMA: a wait for a tile gave up

  const int split = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  if (TMA && tid == 0)   // the descriptor is on its way while the pages are looked up
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&map_run)) : "memory");
  const int G = p.H / p.KV, ps = p.ps;
  // (reserved bit 1) the splits of this (row, key-value head) are one cluster and merge among themselves.  Every way out
  // of the kernel before the cluster's barriers is taken by all blocks of a cluster or by none: they depend on the row alone.
  const bool cluster_merge = (p.reserved & 2) != 0 && p.splits > 1;
  if (p.row_filter == 1 && p.row_q_len[row] != 1) return;   // a row of a prompt: the prefill kernel's
  const RowInfo ri = row_info(p, row);
  const __nv_bfloat16* kv = reinterpret_cast<const __nv_bfloat16*>(p.kv);
  const float* rope = (p.fuse && p.rope_table) ? p.rope_table + (size_t)ri.pos * (HD / 2) * 2 : nullptr;
  if (p.fuse && p.rope_table && ri.pos >= p.rope_positions) {
    if (tid == 0) dk_report(p.err, DK_DEV_BAD_POSITION, ri.t, ri.pos, p.rope_positions);
    return;
  }

  // this block's share of the pages: whole tiles, so that tiles begin where the pool's runs of pages begin
  const int pages_per_tile = TILE / ps;
  const int per = ((ri.n_entries + p.splits - 1) / p.splits + pages_per_tile - 1) / pages_per_tile * pages_per_tile;
  if (per > p.block_entries) {  // more pages than the block table is wide: a wrong table, not a case to compute
    if (tid == 0) dk_report(p.err, DK_DEV_BAD_POSITION, ri.t, ri.pos, p.max_pages * p.ps);
    return;
  }
  const int e_begin = split * per;
  const int e_end = min(ri.n_entries, e_begin + per);
  const int n_tiles = e_end > e_begin ? (e_end - e_begin + pages_per_tile - 1) / pages_per_tile : 0;

  // this block's pages: logical and physical ids, looked up once
  for (int i = tid; i < e_end - e_begin; i += NTHREADS) {
    const int e = e_begin + i;
    const int lp = ri.subset ? ri.sel[e] : ri.first_page + e;
    int page = -1;
    if (lp >= 0 && lp < p.max_pages) {
      page = p.block_table[(size_t)row * p.max_pages + lp];
      if (page < 0 || page >= p.num_pages) {
        dk_report(p.err, DK_DEV_BAD_PAGE, ri.t, lp, page);
        page = -1;
      }
    }
    s_lp[i] = lp;
    s_page[i] = page;
  }
  if (TMA && tid == 0) {
    s_timeout = 0;
    for (int s = 0; s < STAGES; ++s) mbar_init(s2u(&full_bar[s]), 1);   // the one thread that asks for the boxes arrives
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  if (TMA) {
    // which tiles are one run of wholly visible pages
    for (int tile = tid; tile < n_tiles; tile += NTHREADS) {
      const int el0 = tile * pages_per_tile;
      int first = (el0 + pages_per_tile <= e_end - e_begin) ? s_page[el0] : -1;
      for (int k = 0; k < pages_per_tile && first >= 0; ++k) {
        const int lp = s_lp[el0 + k];
        // (the page this launch appends to is fetched the ordinary way: it was just written with ordinary stores)
        if (s_page[el0 + k] != first + k || lp * ps < ri.lo || lp * ps + ps - 1 > ri.pos || (p.fuse == 2 && lp == ri.pos / ps))
          first = -1;
      }
      s_run[tile] = first;
    }
    __syncthreads();
  }

  // Fused append: the block whose share ends with the request's newest page rotates the new
  // token's key, writes key and value to that page, and only then starts to read pages.
  if (p.fuse == 2 && e_end == ri.n_entries && e_end > e_begin) {
    const int page = s_page[e_end - 1 - e_begin];
    if (page >= 0 && s_lp[e_end - 1 - e_begin] == ri.pos / ps) {
      const __nv_bfloat16* krow = reinterpret_cast<const __nv_bfloat16*>(p.q) + (size_t)ri.t * p.q_stride + (size_t)(p.H + kvh) * HD;
      const __nv_bfloat16* vrow = krow + (size_t)p.KV * HD;
      __nv_bfloat16* cache = const_cast<__nv_bfloat16*>(kv);
      const size_t base = ((((size_t)page * 2 + 0) * p.KV + kvh) * ps + ri.pos % ps) * HD;
      if (tid < HD / 2) {
        const float a = __bfloat162float(krow[tid]), b = __bfloat162float(krow[tid + HD / 2]);
        float c = 1.f, sn = 0.f;
        if (rope) {
          c = rope[2 * tid];
          sn = rope[2 * tid + 1];
        }
        cache[base + tid] = __float2bfloat16_rn(a * c - b * sn);
        cache[base + tid + HD / 2] = __float2bfloat16_rn(a * sn + b * c);
      } else if (tid < HD / 2 + HD / 8) {
        const int v8 = tid - HD / 2;
        *reinterpret_cast<uint4*>(cache + base + (size_t)p.KV * ps * HD + v8 * 8) = *reinterpret_cast<const uint4*>(vrow + v8 * 8);
      }
    } else if (tid == 0) {
      dk_report(p.err, DK_DEV_BAD_PAGE, ri.t, ri.pos / ps, page);
    }
    __threadfence();
    __syncthreads();
  }

  // the query heads of this group as A fragments: rows g and g + 8
  uint32_t qa[KB][4];
  {
    const __nv_bfloat16* q = reinterpret_cast<const __nv_bfloat16*>(p.q) + (size_t)ri.t * p.q_stride + (size_t)kvh * G * HD;
#pragma unroll
    for (int kb = 0; kb < KB; ++kb) {
      const int c = kb * 16 + 2 * tq;
      qa[kb][0] = g < G ? *reinterpret_cast<const uint32_t*>(q + (size_t)g * HD + c) : 0u;
      qa[kb][1] = (!LOW && g + 8 < G) ? *reinterpret_cast<const uint32_t*>(q + (size_t)(g + 8) * HD + c) : 0u;
      qa[kb][2] = g < G ? *reinterpret_cast<const uint32_t*>(q + (size_t)g * HD + c + 8) : 0u;
      qa[kb][3] = (!LOW && g + 8 < G) ? *reinterpret_cast<const uint32_t*>(q + (size_t)(g + 8) * HD + c + 8) : 0u;
    }
    if (rope) {
      // pairs (j, j + HD/2): the partner of a fragment of k-block kb sits in k-block kb + KB/2, same register
#pragma unroll
      for (int kb = 0; kb < KB / 2; ++kb) {
#pragma unroll
        for (int hi = 0; hi < 2; ++hi) {           // registers 0,1 (dims c, c+1) and 2,3 (dims c+8, c+9)
          const int j = kb * 16 + 2 * tq + hi * 8;
          const float4 cs = *reinterpret_cast<const float4*>(rope + 2 * j);   // cos j, sin j, cos j+1, sin j+1
#pragma unroll
          for (int r = 0; r < (LOW ? 1 : 2); ++r) {
            __nv_bfloat162 a2 = *reinterpret_cast<__nv_bfloat162*>(&qa[kb][2 * hi + r]);
            __nv_bfloat162 b2 = *reinterpret_cast<__nv_bfloat162*>(&qa[kb + KB / 2][2 * hi + r]);
            const float a0 = __low2float(a2), a1 = __high2float(a2), b0 = __low2float(b2), b1 = __high2float(b2);
            a2 = __floats2bfloat162_rn(a0 * cs.x - b0 * cs.y, a1 * cs.z - b1 * cs.w);
            b2 = __floats2bfloat162_rn(a0 * cs.y + b0 * cs.x, a1 * cs.w + b1 * cs.z);
            qa[kb][2 * hi + r] = *reinterpret_cast<uint32_t*>(&a2);
            qa[kb + KB / 2][2 * hi + r] = *reinterpret_cast<uint32_t*>(&b2);
          }
        }
      }
    }
  }
  // What does not change from tile to tile is worked out once: which key of a tile each of this
  // thread's 16-byte chunks belongs to, where it lands in shared memory, where it sits in a page.
  constexpr int LOADS = TILE * CHUNKS / NTHREADS;
  const int part = tid % CHUNKS;
  int ld_tok[LOADS], ld_pg[LOADS], ld_src[LOADS], ld_dst[LOADS];
#pragma unroll
  for (int i = 0; i < LOADS; ++i) {
    const int tok = (tid + i * NTHREADS) / CHUNKS;
    ld_tok[i] = tok;
    ld_pg[i] = tok / ps;
    ld_src[i] = (tok % ps) * HD + part * 8;                       // elements inside the (page, K, head) block
    ld_dst[i] = (int)tile_offset<HD, TMA>(tok, part);             // bytes inside a K or V tile
  }
  const size_t page_stride = (size_t)2 * p.KV * ps * HD;           // elements from one page to the next
  const size_t v_offset = (size_t)p.KV * ps * HD;                  // from a page's K to its V
  const __nv_bfloat16* kv_head = kv + (size_t)kvh * ps * HD;

  // returns whether every chunk this thread asked for belongs to a key the query may see
  auto load_tile = [&](int tile, int stage) -> bool {
    const uint32_t kdst = smem_u32(kv_smem + (size_t)stage * 2 * TILE_BYTES);
    const uint32_t vdst = kdst + TILE_BYTES;
    const int el0 = tile * pages_per_tile;
    if constexpr (TMA) {
      const int first = s_run[tile];
      if (first >= 0) {       // the same answer in every thread
        if (tid == 0) {
          const uint32_t bar = s2u(&full_bar[stage]);
          mbar_expect_tx(bar, 2u * TILE_BYTES);
#pragma unroll
          for (int half = 0; half < HD / 64; ++half) {
            tma_load_4d(kdst + half * (TILE * 128), &map_run, half * 64, 0, kvh, first, bar);
            tma_load_4d(vdst + half * (TILE * 128), &map_run, half * 64, 0, p.KV + kvh, first, bar);
          }
        }
        return true;
      }
    }
    bool all_valid = true;
#pragma unroll
    for (int i = 0; i < LOADS; ++i) {
      const int el = el0 + ld_pg[i];
      bool valid = false;
      int key = -1;
      const __nv_bfloat16* src = kv_head;
      if (e_begin + el < e_end) {
        const int page = s_page[el];
        const int k = s_lp[el] * ps + (ld_tok[i] % ps);
        if (page >= 0 && k >= ri.lo && k <= ri.pos) {
          valid = true;
          key = k;
          src = kv_head + (size_t)page * page_stride + ld_src[i];
        }
      }
      all_valid &= valid;
      cp_async_16(kdst + ld_dst[i], src, valid);
      cp_async_16(vdst + ld_dst[i], src + v_offset, valid);
      if (part == 0) s_key[stage * TILE + ld_tok[i]] = key;
    }
    return all_valid;
  };

  float o[NT][2 * R];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int c = 0; c < 2 * R; ++c) o[n][c] = 0.f;
  float zd[2] = {0.f, 0.f};                 // accumulators of the empty rows (LOW)
  float m_run[R], l_run[R];                 // rows g (and g + 8): running maximum in log2 units, this thread's part of the row sum
#pragma unroll
  for (int r = 0; r < R; ++r) {
    m_run[r] = -INFINITY;
    l_run[r] = 0.f;
  }
  const float sc_log2 = p.scale * 1.4426950408889634f;

  // full[s]: every key of the tile in stage s is one the query may see, so its scores need no
  // masking.  Each thread knows it for its own chunks; the barriers below collect the votes.
  unsigned full = 0;   // bit s: stage s
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    bool mine = true;
    if (s < n_tiles) mine = load_tile(s, s);
    cp_async_commit();
    if (__syncthreads_and(mine)) full |= 1u << s;
  }
  bool issued_ok = true;
  unsigned tma_parity = 0;   // bit s: parity of the next TMA tile of stage s
  for (int tile = 0; tile < n_tiles; ++tile) {
    cp_async_wait<STAGES - 2>();      // tiles fetched by cp.async (a tile fetched by TMA leaves an empty group)
    if constexpr (TMA) {
      if (s_run[tile] >= 0) {           // fetched by TMA: its stage's barrier tells; the parity of a stage flips with each such tile
        const int st = tile % STAGES;
        if (!mbar_wait(s2u(&full_bar[st]), (tma_parity >> st) & 1u)) s_timeout = 1;
        tma_parity ^= 1u << st;
      }
    }
    {
      // the barrier also tells whether the tile issued in the iteration before is wholly visible
      const bool prev = __syncthreads_and(issued_ok) != 0;
      if (tile > 0) {
        const unsigned bit = 1u << ((tile - 1 + STAGES - 1) % STAGES);
        full = prev ? (full | bit) : (full & ~bit);
      }
      if (TMA && s_timeout) {      // somebody's wait ran out (written before the barrier above): nothing is stored
        if (tid == 0) dk_report(p.err, DK_DEV_TIMEOUT, row, kvh, split);
        if (!cluster_merge) return;
        break;                     // in a cluster the others wait for this block at the barriers: the error is recorded, the output is not to be used
      }
      const int nxt = tile + STAGES - 1;
      issued_ok = true;
      if (nxt < n_tiles) issued_ok = load_tile(nxt, nxt % STAGES);
      cp_async_commit();
    }
    const int stage = tile % STAGES;
    const bool no_mask = ((full >> stage) & 1u) && !ri.dumping;
    const uint32_t kbase = smem_u32(kv_smem + (size_t)stage * 2 * TILE_BYTES);
    const uint32_t vbase = kbase + TILE_BYTES;
    const int* keys = s_key + stage * TILE + warp * 16;

    // S = Q K^T for this warp's 16 keys (two n-tiles of 8)
    float s[2][2 * R];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int c = 0; c < 2 * R; ++c) s[j][c] = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int tok = warp * 16 + j * 8 + (lane & 7);
#pragma unroll
      for (int kb = 0; kb < KB; kb += 2) {
        const int chunk = 2 * kb + (lane >> 3);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, kbase + tile_offset<HD, TMA>(tok, chunk));
        mma_rows<LOW>(s[j], zd, qa[kb], b0, b1);
        mma_rows<LOW>(s[j], zd, qa[kb + 1], b2, b3);
      }
    }
    // mask, dump, online softmax (values in log2 units)
    float tmax[R];
#pragma unroll
    for (int r = 0; r < R; ++r) tmax[r] = -INFINITY;
    if (no_mask) {
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int c = 0; c < 2 * R; ++c) {
          s[j][c] *= sc_log2;
          tmax[c >> 1] = fmaxf(tmax[c >> 1], s[j][c]);
        }
    } else {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int key = keys[j * 8 + 2 * tq + c];
#pragma unroll
          for (int r = 0; r < R; ++r) {
            float v = s[j][2 * r + c];
            if (key < 0) {
              v = -INFINITY;
            } else {
              if (ri.dumping && key < p.dump_stride && g + 8 * r < G)
                p.dump[((size_t)row * p.H + kvh * G + g + 8 * r) * p.dump_stride + key] = v * p.scale;
              v *= sc_log2;
            }
            s[j][2 * r + c] = v;
            tmax[r] = fmaxf(tmax[r], v);
          }
        }
      }
    }
    float corr[R], m_use[R];
    bool moved = false;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
      tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
      const float m_new = fmaxf(m_run[r], tmax[r]);
      m_use[r] = m_new == -INFINITY ? 0.f : m_new;   // a warp whose 16 keys are all masked
      corr[r] = m_run[r] == -INFINITY ? 0.f : exp2f(m_run[r] - m_use[r]);
      moved |= corr[r] != 1.f;
      m_run[r] = m_new;
      l_run[r] *= corr[r];
    }
    uint32_t pa[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float p0 = exp2f(s[j][2 * r] - m_use[r]), p1 = exp2f(s[j][2 * r + 1] - m_use[r]);
        l_run[r] += p0 + p1;
        pa[2 * j + r] = pack_bf16(p0, p1);
      }
    // O = O * corr + P V; once the maxima have settled corr is 1 and the scaling is skipped
    if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int c = 0; c < 2 * R; ++c) o[n][c] *= corr[c >> 1];
    }
    {
      const int tok = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int n = 0; n < NT; n += 2) {
        const int chunk = n + (lane >> 4);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, vbase + tile_offset<HD, TMA>(tok, chunk));
        mma_rows<LOW>(o[n], zd, pa, b0, b1);
        mma_rows<LOW>(o[n + 1], zd, pa, b2, b3);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // merge the four warps through shared memory (the tiles are no longer needed)
#pragma unroll
  for (int r = 0; r < R; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  float* w_o = reinterpret_cast<float*>(smem);         // [NWARPS][16][HD]
  float* w_m = w_o + NWARPS * 16 * HD;                 // [NWARPS][16]
  float* w_l = w_m + NWARPS * 16;                      // [NWARPS][16]
  float* c_o = w_l + NWARPS * 16;                      // cluster merge: this block's [G][HD] output, then {m, l} per row
  float* c_ml = c_o + 16 * HD;
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    float* base = w_o + ((size_t)warp * 16) * HD + n * 8 + 2 * tq;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      base[(size_t)(g + 8 * r) * HD] = o[n][2 * r];
      base[(size_t)(g + 8 * r) * HD + 1] = o[n][2 * r + 1];
    }
  }
  if (tq == 0) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      w_m[warp * 16 + g + 8 * r] = m_run[r];
      w_l[warp * 16 + g + 8 * r] = l_run[r];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < G * HD; idx += NTHREADS) {
    const int r = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, w_m[w * 16 + r]);
    float L = 0.f, acc = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < NWARPS; ++w) {
        const float mw = w_m[w * 16 + r];
        const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
        L += w_l[w * 16 + r] * f;
        acc += w_o[((size_t)w * 16 + r) * HD + d] * f;
      }
    }
    const int h = kvh * G + r;
    if (p.splits == 1) {
      reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)ri.t * p.H * HD + (size_t)h * HD + d] =
          __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
      if (p.lse != nullptr && d == 0) p.lse[(size_t)ri.t * p.H + h] = L > 0.f ? fmaf(M, 0.6931471805599453f, logf(L)) : -INFINITY;
    } else if (cluster_merge) {
      c_o[idx] = acc;
      if (d == 0) {
        c_ml[2 * r] = M;
        c_ml[2 * r + 1] = L;
      }
    } else {
      float* sc = reinterpret_cast<float*>(p.scratch);
      sc[part_o_index(p, row, h, split, HD) + d] = acc;
      if (d == 0) {
        sc[part_ml_index(p, row, h, split)] = M;
        sc[part_ml_index(p, row, h, split) + 1] = L;
      }
    }
  }
  if (cluster_merge) {
    // Block `split` of the cluster merges its share of the [G][HD] outputs from all blocks' shared memory, in split
    // order and with the arithmetic of the merge kernel below (so both ways give the same bits).
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const int S = p.splits;                 // 2..8, the cluster's size
    const int total = G * HD;
    const int share = (total + S - 1) / S;
    const int end = min(total, (split + 1) * share);
    const float* ro[8];
    const float* rml[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      ro[j] = j < S ? cluster.map_shared_rank(c_o, j) : c_o;
      rml[j] = j < S ? cluster.map_shared_rank(c_ml, j) : c_ml;
    }
    for (int idx = split * share + tid; idx < end; idx += NTHREADS) {
      const int r = idx / HD, d = idx % HD;
      float m[8], l[8], o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool ok = j < S;
        m[j] = ok ? rml[j][2 * r] : -INFINITY;
        l[j] = ok ? rml[j][2 * r + 1] : 0.f;
        o[j] = ok ? ro[j][idx] : 0.f;
      }
      float M = -INFINITY, L = 0.f, acc = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) M = fmaxf(M, m[j]);
      if (M != -INFINITY) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float f = m[j] == -INFINITY ? 0.f : exp2f(m[j] - M);
          L += l[j] * f;
          acc += o[j] * f;
        }
      }
      const int h = kvh * G + r;
      reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)ri.t * p.H * HD + (size_t)h * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
      if (p.lse != nullptr && d == 0) p.lse[(size_t)ri.t * p.H + h] = L > 0.f ? fmaf(M, 0.6931471805599453f, logf(L)) : -INFINITY;
    }
    cluster.sync();                           // nobody leaves while its shared memory is still read
  }
}

// Merges the splits of one (row, head) in split order.
template <int HD>
__global__ void attention_decode_merge_kernel(const DkAttnParams p) {
  const int row = blockIdx.y, h = blockIdx.x, d = threadIdx.x;
  if (p.row_filter == 1 && p.row_q_len[row] != 1) return;
  const float* sc = reinterpret_cast<const float*>(p.scratch);
  const int t = p.row_q_start[row] + p.row_q_len[row] - 1;
  // Sixteen splits at a time: their maxima, sums and outputs are asked for together (one round
  // trip to the L2 instead of one per split), then added in split order; a later group rescales
  // what the groups before it added.
  constexpr int GROUP = 16;
  const float* ml = sc + part_ml_index(p, row, h, 0);          // {m, l} of split s at ml[2 s]
  const float* po = sc + part_o_index(p, row, h, 0, HD) + (d < HD ? d : 0);   // this thread's output of split s at po[s HD]
  float M = -INFINITY, L = 0.f, acc = 0.f;
  for (int s0 = 0; s0 < p.splits; s0 += GROUP) {
    float m[GROUP], l[GROUP], o[GROUP];
#pragma unroll
    for (int j = 0; j < GROUP; ++j) {
      const int s = s0 + j;
      const bool ok = s < p.splits;
      m[j] = ok ? ml[2 * s] : -INFINITY;
      l[j] = ok ? ml[2 * s + 1] : 0.f;
      o[j] = ok ? po[(size_t)s * HD] : 0.f;
    }
    float group_max = M;
#pragma unroll
    for (int j = 0; j < GROUP; ++j) group_max = fmaxf(group_max, m[j]);
    if (group_max != -INFINITY) {
      const float keep = M == -INFINITY ? 0.f : exp2f(M - group_max);
      L *= keep;
      acc *= keep;
#pragma unroll
      for (int j = 0; j < GROUP; ++j) {
        const float f = m[j] == -INFINITY ? 0.f : exp2f(m[j] - group_max);
        L += l[j] * f;
        acc += o[j] * f;
      }
      M = group_max;
    }
  }
  if (d < HD)
    reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)t * p.H * HD + (size_t)h * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
  if (p.lse != nullptr && d == 0) p.lse[(size_t)t * p.H + h] = L > 0.f ? fmaf(M, 0.6931471805599453f, logf(L)) : -INFINITY;
}

// Raises the kernel's limit of dynamic shared memory to ``smem`` bytes on the current device when it is
// lower (the attribute belongs to the device's copy of the kernel; setting it anew would also lower it).
template <int HD, bool LOW, bool TMA>
int configure(size_t smem) {
  static size_t configured_on[DK_MAX_DEVICES] = {0};
  size_t& configured = configured_on[dk_current_device()];
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<HD, LOW, TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      dk_set_error("attention_decode: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      return DK_ERR_LAUNCH;
    }
    configured = smem;
  }
  return 0;
}

template <int HD, bool LOW, bool TMA>
int launch(const DkAttnParams& pin, cudaStream_t stream) {
  DkAttnParams p = pin;
  // entries (pages) one block can be given: the widest request split evenly, in whole tiles
  const int pages_per_tile = TILE / p.ps > 0 ? TILE / p.ps : 1;
  p.block_entries = ((p.max_pages + p.splits - 1) / p.splits + pages_per_tile - 1) / pages_per_tile * pages_per_tile;
  if (p.block_entries > 8192) {
    dk_set_error("attention_decode: %d pages per block are above the 8192 it keeps in shared memory; use more splits", p.block_entries);
    return DK_ERR_ARG;
  }
  const size_t tile_bytes = (size_t)STAGES * 2 * TILE * HD * 2 + (size_t)STAGES * TILE * sizeof(int) + (size_t)3 * p.block_entries * sizeof(int);
  constexpr size_t merge_bytes = (size_t)NWARPS * 16 * HD * sizeof(float) + 2 * NWARPS * 16 * sizeof(float) + (size_t)16 * HD * sizeof(float) + 32 * sizeof(float);
  const size_t smem = (tile_bytes > merge_bytes ? tile_bytes : merge_bytes) + (TMA ? 1024 : 0);
  CUtensorMap map_run;
  memset(&map_run, 0, sizeof(map_run));
  if (TMA) {
    // the cache as [page][K|V, head][offset][hd]: a run of pages of one head in one box of a tile's pages
    const unsigned long long dims[4] = {(unsigned long long)HD, (unsigned long long)p.ps, (unsigned long long)(2 * p.KV),
                                        (unsigned long long)p.num_pages};
    const unsigned long long strides[3] = {(unsigned long long)HD * 2, (unsigned long long)p.ps * HD * 2,
                                           (unsigned long long)2 * p.KV * p.ps * HD * 2};
    DK_REQUIRE(make_tensor_map_bf16_4d(&map_run, p.kv, dims, strides, p.ps, TILE / p.ps),
               "attention_decode: cannot encode the tensor map of runs of pages");
  }
  if (int rc = configure<HD, LOW, TMA>(smem)) return rc;
  dim3 grid(p.splits, p.KV, p.rows);
  if ((p.reserved & 2) != 0 && p.splits > 1) {
    // the splits of a (row, key-value head) as one cluster, which merges them itself
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_decode_kernel<HD, LOW, TMA>, map_run, p);
    if (e != cudaSuccess) {
      dk_set_error("attention_decode: launch of clusters of %d blocks failed: %s", p.splits, cudaGetErrorString(e));
      return DK_ERR_LAUNCH;
    }
    return dk_check_launch("attention_decode");
  }
  attention_decode_kernel<HD, LOW, TMA><<<grid, NTHREADS, smem, stream>>>(map_run, p);
  int rc = dk_check_launch("attention_decode");
  if (rc != 0 || p.splits == 1) return rc;
  dim3 mgrid(p.H, p.rows);
  attention_decode_merge_kernel<HD><<<mgrid, HD, 0, stream>>>(p);
  return dk_check_launch("attention_decode_merge");
}
}  // namespace

// Floats of scratch that a launch with these sizes needs (0 when splits == 1).
extern "C" long long dk_attention_decode_scratch_floats(int rows, int H, int hd, int splits) {
  if (splits <= 1) return 0;
  return (long long)rows * H * splits * (hd + 2);
}

// Blocks of the decode kernel that one SM holds at once for these sizes (registers and shared
// memory decide), asked of the runtime for the current device; 0 with the error set on failure.
extern "C" int dk_attention_decode_blocks_per_sm(int H, int KV, int hd, int block_entries) {
  if (KV <= 0 || (hd != 64 && hd != 128)) return 0;
  const size_t tile_bytes = (size_t)STAGES * 2 * TILE * hd * 2 + (size_t)STAGES * TILE * sizeof(int) + (size_t)3 * block_entries * sizeof(int);
  const size_t merge_bytes = (size_t)NWARPS * 16 * hd * sizeof(float) + 2 * NWARPS * 16 * sizeof(float) + (size_t)16 * hd * sizeof(float) + 32 * sizeof(float);
  const size_t smem = tile_bytes > merge_bytes ? tile_bytes : merge_bytes;
  const bool low = H / KV <= 8;
  int n = 0, rc;
  cudaError_t e;
  if (hd == 64 && low) {
    rc = configure<64, true, false>(smem);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attention_decode_kernel<64, true, false>, NTHREADS, smem);
  } else if (hd == 64) {
    rc = configure<64, false, false>(smem);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attention_decode_kernel<64, false, false>, NTHREADS, smem);
  } else if (low) {
    rc = configure<128, true, false>(smem);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attention_decode_kernel<128, true, false>, NTHREADS, smem);
  } else {
    rc = configure<128, false, false>(smem);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attention_decode_kernel<128, false, false>, NTHREADS, smem);
  }
  if (rc != 0) return 0;
  if (e != cudaSuccess) {
    dk_set_error("attention_decode: occupancy query failed: %s", cudaGetErrorString(e));
    return 0;
  }
  return n;
}

// Clusters of ``splits`` blocks of the decode kernel that the device holds at once (a cluster needs all its blocks
// resident in one GPC at the same time, so this is less than blocks per SM x SMs / splits); 0 with the error set on failure.
extern "C" int dk_attention_decode_max_clusters(int H, int KV, int hd, int block_entries, int splits) {
  if (KV <= 0 || (hd != 64 && hd != 128) || splits < 1 || splits > 8) return 0;
  const size_t tile_bytes = (size_t)STAGES * 2 * TILE * hd * 2 + (size_t)STAGES * TILE * sizeof(int) + (size_t)3 * block_entries * sizeof(int);
  const size_t merge_bytes = (size_t)NWARPS * 16 * hd * sizeof(float) + 2 * NWARPS * 16 * sizeof(float) + (size_t)16 * hd * sizeof(float) + 32 * sizeof(float);
  const size_t smem = tile_bytes > merge_bytes ? tile_bytes : merge_bytes;
  const bool low = H / KV <= 8;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(splits, 1, 1);
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0, rc;
  cudaError_t e;
  if (hd == 64 && low) {
    rc = configure<64, true, false>(smem);
    e = cudaOccupancyMaxActiveClusters(&n, attention_decode_kernel<64, true, false>, &cfg);
  } else if (hd == 64) {
    rc = configure<64, false, false>(smem);
    e = cudaOccupancyMaxActiveClusters(&n, attention_decode_kernel<64, false, false>, &cfg);
  } else if (low) {
    rc = configure<128, true, false>(smem);
    e = cudaOccupancyMaxActiveClusters(&n, attention_decode_kernel<128, true, false>, &cfg);
  } else {
    rc = configure<128, false, false>(smem);
    e = cudaOccupancyMaxActiveClusters(&n, attention_decode_kernel<128, false, false>, &cfg);
  }
  if (rc != 0) return 0;
  if (e != cudaSuccess) {
    dk_set_error("attention_decode: cluster occupancy query failed: %s", cudaGetErrorString(e));
    return 0;
  }
  return n;
}

// 1 when the fast kernel takes these sizes, else 0 (the caller then uses the plain kernel).
extern "C" int dk_attention_decode_supported(int dtype, int H, int KV, int hd, int ps) {
  if (dtype != DK_BF16 || KV <= 0 || H % KV != 0) return 0;
  if (H / KV > 16) return 0;
  if (hd != 64 && hd != 128) return 0;
  if (ps < 1 || ps > TILE || (ps & (ps - 1)) != 0) return 0;
  return 1;
}

extern "C" int dk_attention_decode(const DkAttnParams* pp, cudaStream_t stream) {
  const DkAttnParams& p = *pp;
  if (p.rows == 0) return 0;
  DK_REQUIRE(dk_attention_decode_supported(p.dtype, p.H, p.KV, p.hd, p.ps),
             "attention_decode: sizes not taken (bfloat16, head size 64 or 128, at most 16 query heads per key-value head, "
             "page size a power of two <= 64): dtype=%d H=%d KV=%d hd=%d ps=%d", p.dtype, p.H, p.KV, p.hd, p.ps);
  DK_REQUIRE(p.T == p.rows || p.row_filter == 1,
             "attention_decode: %d tokens for %d rows; every row must bring one token unless rows are filtered", p.T, p.rows);
  DK_REQUIRE(p.row_q_start != nullptr && p.row_q_len != nullptr, "attention_decode: row_q_start / row_q_len are missing");
  DK_REQUIRE(p.splits >= 1 && p.splits <= 65535 && p.KV <= 65535 && p.rows <= 65535, "attention_decode: grid too large");
  DK_REQUIRE((p.reserved & 2) == 0 || p.splits <= 8, "attention_decode: a cluster merges at most 8 splits, not %d", p.splits);
  DK_REQUIRE(p.splits == 1 || (p.reserved & 2) != 0 || p.scratch != nullptr, "attention_decode: %d splits need a scratch buffer", p.splits);
  DK_REQUIRE(p.q_stride % 2 == 0, "attention_decode: q stride must be even");
  DK_REQUIRE(p.fuse >= 0 && p.fuse <= 2, "attention_decode: fuse must be 0, 1 or 2");
  DK_REQUIRE(p.fuse == 0 || p.q_stride >= (p.H + 2 * p.KV) * p.hd,
             "attention_decode: with fuse the query rows must be [q | k | v] rows of width %d, the stride is %d", (p.H + 2 * p.KV) * p.hd, p.q_stride);
  DK_REQUIRE(p.fuse == 0 || p.rope_table == nullptr || p.rope_positions > 0, "attention_decode: a rope table without rows");
  DK_REQUIRE(p.sel_pages == nullptr || (p.sel_count != nullptr && p.row_flags != nullptr && p.row_slot != nullptr),
             "attention_decode: chosen pages are given without their counts, row flags or slots");
  const bool low = p.H / p.KV <= 8;
  // the TMA variant: pages of at least 8 tokens (a page is a multiple of the swizzle's 8 rows), no score
  // dump (a dump needs every key's position), a cache that starts on a 16-byte boundary
  // and a caller that has not said (reserved bit 0) that its pages lie scattered: then no tile is a run,
  // and the cp.async path of the TMA variant is the slower one (measured: 122 against 111 us)
  const bool tma = p.ps >= 8 && p.dump == nullptr && ((uintptr_t)p.kv % 16) == 0 && (p.reserved & 1) == 0;
  if (p.hd == 64) {
    if (tma) return low ? launch<64, true, true>(p, stream) : launch<64, false, true>(p, stream);
    return low ? launch<64, true, false>(p, stream) : launch<64, false, false>(p, stream);
  }
  if (tma) return low ? launch<128, true, true>(p, stream) : launch<128, false, true>(p, stream);
  return low ? launch<128, true, false>(p, stream) : launch<128, false, false>(p, stream);
}

// --------------------------------------------------------------------------------------
// The same launch with its scratch inside the library, for callers that cannot allocate
// (see no_alloc.h).  In host code the name of a __device__ array is only a handle for the
// runtime, not an address a kernel can use, so the address is asked for once per device.
#include "no_alloc.h"
#include <mutex>

static __device__ __align__(256) float g_static_scratch[DK_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_static_scratch_addr[MAX_DEVICES] = {nullptr};
std::mutex g_static_scratch_mutex;

// Device address of the built-in scratch on the current device, or nullptr with the error set.
float* static_scratch_address() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
    dk_set_error("attention_decode_static: cannot tell the current device (%s)", cudaGetErrorString(e));
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_addr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      dk_set_error("attention_decode_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      return nullptr;
    }
    g_static_scratch_addr[dev] = ptr;
  }
  return g_static_scratch_addr[dev];
}
}  // namespace

extern "C" int dk_attention_decode_static(const DkAttnParams* pp, cudaStream_t stream) {
  DK_REQUIRE(pp != nullptr, "attention_decode_static: no parameters");
  DkAttnParams p = *pp;
  p.scratch = nullptr;
  p.reserved &= ~2;          // the splits go through the built-in scratch here, not through a cluster
  if (p.rows == 0) return 0;
  const long long need = dk_attention_decode_scratch_floats(p.rows, p.H, p.hd, p.splits);
  DK_REQUIRE(need <= (long long)DK_STATIC_SCRATCH_FLOATS,
             "attention_decode_static: %d rows x %d heads x %d splits x head size %d need %lld floats of scratch, the "
             "built-in buffer holds %d; use fewer splits or rows, or dk_attention_decode with a buffer of your own",
             p.rows, p.H, p.splits, p.hd, need, (int)DK_STATIC_SCRATCH_FLOATS);
  if (p.splits > 1) {
    float* addr = static_scratch_address();
    if (addr == nullptr) return DK_ERR_LAUNCH;
    p.scratch = addr;
  }
  return dk_attention_decode(&p, stream);
}
