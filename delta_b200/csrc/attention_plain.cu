// Plain paged attention: one block per (token, head), any number of new tokens
// per request, causal, over the block table.  It handles every case the engine
// has (whole cache, a window of it, a list of chosen pages, the dump of scaled
// scores for DELTA's page scoring) in the simplest form, float arithmetic
// throughout.  The faster kernels are checked against this one.
//
//   s[t]  = (q . k[t]) * scale  for keys  lo <= t <= pos            (backend.py:542, 1103)
//   y     = sum_t softmax(s)[t] * v[t]
#include "common.cuh"
#include "attention_params.h"

extern "C" int dk_sizeof_attn_params() { return (int)sizeof(DkAttnParams); }

namespace {
constexpr int CH = 128;  // key slots per pass = threads per block

template <typename T>
__global__ void __launch_bounds__(CH) attention_plain_kernel(const DkAttnParams p) {
  extern __shared__ float smem[];
  float* qs = smem;               // hd
  float* sc = qs + p.hd;          // CH
  float* scratch = sc + CH;       // 33
  long long* voff = (long long*)(scratch + 34 + ((p.hd + CH + 34) & 1));  // CH, 8-byte aligned
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int row = p.tok_row[t], pos = p.tok_pos[t];
  const int hd = p.hd, ps = p.ps, KV = p.KV;
  const int g = h / (p.H / KV);
  const T* q = (const T*)p.q + (size_t)t * p.q_stride + (size_t)h * hd;
  const T* kv = (const T*)p.kv;
  for (int i = tid; i < hd; i += CH) qs[i] = to_f32<T>(q[i]);

  const int flags = p.row_flags ? p.row_flags[row] : 0;
  const int slot = p.row_slot ? p.row_slot[row] : row;
  int n_sel = -1;
  if (p.sel_pages != nullptr && (flags & 1)) n_sel = p.sel_count[slot];
  const bool subset = n_sel >= 0;
  const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
  const int first_page = lo / ps;
  const int n_entries = subset ? n_sel : (pos / ps - first_page + 1);
  const int* sel = subset ? p.sel_pages + (size_t)slot * p.sel_stride : nullptr;
  const bool dumping = p.dump != nullptr && (flags & 1);
  float* dump = dumping ? p.dump + ((size_t)row * p.H + h) * p.dump_stride : nullptr;

  float m = -INFINITY, l = 0.f;
  float acc[2] = {0.f, 0.f};
  const int pages_per_pass = CH / ps;
  __syncthreads();

  for (int e0 = 0; e0 < n_entries; e0 += pages_per_pass) {
    const int e = e0 + tid / ps, off = tid % ps;
    float s = -INFINITY;
    long long vo = -1;
    if (e < n_entries) {
      const int lp = subset ? sel[e] : first_page + e;
      const int key = lp * ps + off;
      if (lp >= 0 && lp < p.max_pages && key >= lo && key <= pos) {
        const int page = p.block_table[(size_t)row * p.max_pages + lp];
        if (page < 0 || page >= p.num_pages) {
          dk_report(p.err, DK_DEV_BAD_PAGE, t, lp, page);
        } else {
          const T* kr = kv + ((((size_t)page * 2 + 0) * KV + g) * ps + off) * hd;
          float d = 0.f;
          for (int i = 0; i < hd; ++i) d = fmaf(qs[i], to_f32<T>(kr[i]), d);
          s = d * p.scale;
          vo = (long long)((((size_t)page * 2 + 1) * KV + g) * ps + off) * hd;
          if (dumping && key < p.dump_stride) dump[key] = s;
        }
      }
    }
    voff[tid] = vo;
    const float cmax = block_max(s, scratch);
    if (cmax == -INFINITY) {
      __syncthreads();
      continue;
    }
    const float m_new = fmaxf(m, cmax);
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float pr = (vo >= 0) ? expf(s - m_new) : 0.f;
    sc[tid] = pr;
    const float psum = block_sum(pr, scratch);
    l = l * corr + psum;
    m = m_new;
#pragma unroll
    for (int dd = 0; dd < 2; ++dd) {
      const int d = tid + dd * CH;
      if (d < hd) {
        float a = acc[dd] * corr;
        for (int k = 0; k < CH; ++k) {
          const long long o = voff[k];
          if (o >= 0) a = fmaf(sc[k], to_f32<T>(kv[o + d]), a);
        }
        acc[dd] = a;
      }
    }
    __syncthreads();
  }
  T* out = (T*)p.out + (size_t)t * p.H * hd + (size_t)h * hd;
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int dd = 0; dd < 2; ++dd) {
    const int d = tid + dd * CH;
    if (d < hd) out[d] = from_f32<T>(acc[dd] * inv);
  }
  if (p.lse != nullptr && tid == 0) p.lse[(size_t)t * p.H + h] = l > 0.f ? m + logf(l) : -INFINITY;
}
}  // namespace

extern "C" int dk_attention_plain(const DkAttnParams* pp, cudaStream_t stream) {
  const DkAttnParams& p = *pp;
  if (p.T == 0) return 0;
  DK_REQUIRE(p.T > 0 && p.H > 0 && p.KV > 0 && p.hd > 0, "attention: bad sizes T=%d H=%d KV=%d hd=%d", p.T, p.H, p.KV, p.hd);
  DK_REQUIRE(p.H % p.KV == 0, "attention: %d heads are no multiple of %d key-value heads", p.H, p.KV);
  DK_REQUIRE(p.hd <= 2 * CH, "attention: head size %d is above the %d this kernel takes", p.hd, 2 * CH);
  DK_REQUIRE(p.ps >= 1 && p.ps <= CH && (p.ps & (p.ps - 1)) == 0, "attention: page size %d must be a power of two <= %d", p.ps, CH);
  DK_REQUIRE(p.H <= 65535, "attention: too many heads");
  DK_REQUIRE(p.sel_pages == nullptr || (p.sel_count != nullptr && p.row_flags != nullptr && p.row_slot != nullptr),
             "attention: chosen pages are given without their counts, row flags or slots");
  DK_REQUIRE(p.dump == nullptr || p.row_flags != nullptr, "attention: a score dump is asked for without row flags");
  const size_t smem = (size_t)(p.hd + CH + 36) * sizeof(float) + (size_t)CH * sizeof(long long);
  dim3 grid(p.T, p.H);
  if (p.dtype == DK_F32) attention_plain_kernel<float><<<grid, CH, smem, stream>>>(p);
  else if (p.dtype == DK_BF16) attention_plain_kernel<__nv_bfloat16><<<grid, CH, smem, stream>>>(p);
  else DK_REQUIRE(false, "attention: unknown dtype %d", p.dtype);
  return dk_check_launch("attention_plain");
}
