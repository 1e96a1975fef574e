// Embedding gather, RMSNorm (with the residual add fused in front of it), SwiGLU
// gate, and rotary positions fused with the append of keys and values to the
// paged cache.  All of them are bound by memory traffic; each reads its input
// once and writes its output once.
#include "common.cuh"
#include <stdarg.h>

static thread_local char g_last_error[512] = "";
extern "C" const char* dk_last_error() { return g_last_error; }
void dk_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

// ---------------------------------------------------------------- embedding
// out[t, :] = table[tokens[t], :]          (reference: model.py:199)
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ tokens, const T* __restrict__ table, T* __restrict__ out,
                                 int d, int vocab, int* err) {
  const int t = blockIdx.x;
  const int tok = tokens[t];
  if (tok < 0 || tok >= vocab) {
    if (threadIdx.x == 0) dk_report(err, DK_DEV_BAD_TOKEN, t, tok, vocab);
    for (int i = threadIdx.x; i < d; i += blockDim.x) out[(size_t)t * d + i] = from_f32<T>(0.f);
    return;
  }
  const T* src = table + (size_t)tok * d;
  T* dst = out + (size_t)t * d;
  constexpr int VEC = 16 / sizeof(T);
  if ((d % VEC) == 0) {  // rows start on 16-byte boundaries then
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int i = threadIdx.x; i < d / VEC; i += blockDim.x) d4[i] = s4[i];
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = src[i];
  }
}

extern "C" int dk_embedding(const int* tokens, const void* table, void* out, int T_, int d, int vocab, int dtype,
                            int* err, cudaStream_t stream) {
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && d > 0 && vocab > 0, "embedding: bad sizes T=%d d=%d vocab=%d", T_, d, vocab);
  const int threads = d >= 1024 ? 256 : 128;
  if (dtype == DK_F32)
    embedding_kernel<float><<<T_, threads, 0, stream>>>(tokens, (const float*)table, (float*)out, d, vocab, err);
  else if (dtype == DK_BF16)
    embedding_kernel<__nv_bfloat16><<<T_, threads, 0, stream>>>(tokens, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, d, vocab, err);
  else
    DK_REQUIRE(false, "embedding: unknown dtype %d", dtype);
  return dk_check_launch("embedding");
}

// ------------------------------------------------------------------ RMSNorm
// For output row r, source row s = rows ? rows[r] : r.
//   if add != nullptr:  x[s] <- x[s] + add[s]      (sum in float, stored in T)
//   n = x[s] * rsqrt(mean(x[s]^2) + eps)           (float)
//   out[r] = cast_first ? T(n) * w : n * w         (reference casts first: model.py:531-532)
// W is the type of the weight, which a model folder may store in 32 bit.
template <typename T, typename W>
__global__ void rms_norm_kernel(T* __restrict__ x, const T* __restrict__ add, const W* __restrict__ w, T* __restrict__ out,
                                const int* __restrict__ rows, int d, float eps, int cast_first) {
  extern __shared__ float row[];  // d floats + 33 for the reduction
  float* scratch = row + d;
  const int r = blockIdx.x;
  const int s = rows ? rows[r] : r;
  T* xs = x + (size_t)s * d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = to_f32<T>(xs[i]);
    if (add) {
      v += to_f32<T>(add[(size_t)s * d + i]);
      const T stored = from_f32<T>(v);
      xs[i] = stored;
      v = to_f32<T>(stored);
    }
    row[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)d + eps);
  T* o = out + (size_t)r * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float n = row[i] * inv;
    if (cast_first) n = to_f32<T>(from_f32<T>(n));
    o[i] = from_f32<T>(n * to_f32<W>(w[i]));
  }
}

// The same with 16-byte loads and stores; used when the width is a multiple of the vector
// length.  Every thread first loads all its vectors, so the loads are in flight together.
template <typename T, typename W, int MAXV>
__global__ void rms_norm_vec_kernel(T* __restrict__ x, const T* __restrict__ add, const W* __restrict__ w, T* __restrict__ out,
                                    const int* __restrict__ rows, int d, float eps, int cast_first) {
  constexpr int VEC = 16 / sizeof(T);
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int s = rows ? rows[r] : r;
  const int nvec = d / VEC;
  uint4* x4 = reinterpret_cast<uint4*>(x + (size_t)s * d);
  const uint4* a4 = add ? reinterpret_cast<const uint4*>(add + (size_t)s * d) : nullptr;
  uint4 xv[MAXV], av[MAXV];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      xv[i] = x4[v];
      if (a4) av[i] = a4[v];
    }
  }
  float vals[MAXV][VEC];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      const T* xe = reinterpret_cast<const T*>(&xv[i]);
      const T* ae = reinterpret_cast<const T*>(&av[i]);
      uint4 st;
      T* se = reinterpret_cast<T*>(&st);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        float f = to_f32<T>(xe[e]);
        if (a4) {
          f += to_f32<T>(ae[e]);
          se[e] = from_f32<T>(f);
          f = to_f32<T>(se[e]);
        }
        vals[i][e] = f;
        ss += f * f;
      }
      if (a4) x4[v] = st;
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)d + eps);
  uint4* o4 = reinterpret_cast<uint4*>(out + (size_t)r * d);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      uint4 st;
      T* se = reinterpret_cast<T*>(&st);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        float n = vals[i][e] * inv;
        if (cast_first) n = to_f32<T>(from_f32<T>(n));
        se[e] = from_f32<T>(n * to_f32<W>(w[(size_t)v * VEC + e]));
      }
      o4[v] = st;
    }
  }
}

extern "C" int dk_rms_norm(void* x, const void* add, const void* w, void* out, const int* rows, int n_rows, int d,
                           float eps, int dtype, int w_dtype, int cast_first, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  DK_REQUIRE(n_rows > 0 && d > 0, "rms_norm: bad sizes rows=%d d=%d", n_rows, d);
  DK_REQUIRE(d <= 12000, "rms_norm: width %d is above the 12000 this kernel keeps in shared memory", d);
  // few rows (a decode step): many threads per row shorten the one pass every block makes; many rows
  // (a prompt): two vectors per thread and more blocks per SM carry more bytes (measured, width 4096)
  const int threads = d >= 2048 ? ((n_rows >= 256 && d >= 4096) ? 256 : 512) : (d >= 512 ? 256 : 128);
  const size_t smem = (size_t)(d + 33) * sizeof(float);
  const int vec = dtype == DK_BF16 ? 8 : 4;
  const bool use_vec = (d % vec) == 0 && d / vec <= 2 * threads;
#define LAUNCH(T, W)                                                                                                          \
  do {                                                                                                                        \
    if (use_vec)                                                                                                              \
      rms_norm_vec_kernel<T, W, 2><<<n_rows, threads, 0, stream>>>((T*)x, (const T*)add, (const W*)w, (T*)out, rows, d, eps, cast_first); \
    else                                                                                                                      \
      rms_norm_kernel<T, W><<<n_rows, threads, smem, stream>>>((T*)x, (const T*)add, (const W*)w, (T*)out, rows, d, eps, cast_first); \
  } while (0)
  if (dtype == DK_F32 && w_dtype == DK_F32) LAUNCH(float, float);
  else if (dtype == DK_BF16 && w_dtype == DK_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == DK_BF16 && w_dtype == DK_F32) LAUNCH(__nv_bfloat16, float);
  else DK_REQUIRE(false, "rms_norm: unsupported dtypes x=%d w=%d", dtype, w_dtype);
#undef LAUNCH
  return dk_check_launch("rms_norm");
}

// ------------------------------------------------------------- SwiGLU gate
// gu[t, 0:I] = gate, gu[t, I:2I] = up;  out[t, i] = silu(gate) * up
// (reference: model.py:514; computed in float, rounded once)
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total) {
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = to_f32<T>(gu[t * 2 * I + i]);
    const float u = to_f32<T>(gu[t * 2 * I + I + i]);
    const float s = g / (1.f + expf(-g));
    out[idx] = from_f32<T>(s * u);
  }
}

// The same with 16-byte loads and stores, for I a multiple of the vector length: blockIdx.y walks
// the tokens, the threads of blockIdx.x the vectors of a token, so no index is divided.
template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, int T_) {
  constexpr int VEC = 16 / sizeof(T);
  const int nvec = I / VEC;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= nvec) return;
  for (int t = blockIdx.y; t < T_; t += gridDim.y) {
    const uint4* row = reinterpret_cast<const uint4*>(gu + (size_t)t * 2 * I);
    const uint4 g4 = row[v], u4 = row[nvec + v];
    const T* ge = reinterpret_cast<const T*>(&g4);
    const T* ue = reinterpret_cast<const T*>(&u4);
    uint4 o4;
    T* oe = reinterpret_cast<T*>(&o4);
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      const float g = to_f32<T>(ge[e]);
      oe[e] = from_f32<T>(g / (1.f + expf(-g)) * to_f32<T>(ue[e]));
    }
    reinterpret_cast<uint4*>(out + (size_t)t * I)[v] = o4;
  }
}

extern "C" int dk_silu_mul(const void* gu, void* out, int T_, int I, int dtype, cudaStream_t stream) {
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && I > 0, "silu_mul: bad sizes T=%d I=%d", T_, I);
  DK_REQUIRE(dtype == DK_F32 || dtype == DK_BF16, "silu_mul: unknown dtype %d", dtype);
  const int vec = dtype == DK_BF16 ? 8 : 4;
  const int threads = 256;
  if ((I % vec) == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)out % 16) == 0) {
    dim3 grid((I / vec + threads - 1) / threads, T_ < 32768 ? T_ : 32768);
    if (dtype == DK_F32)
      silu_mul_vec_kernel<float><<<grid, threads, 0, stream>>>((const float*)gu, (float*)out, I, T_);
    else
      silu_mul_vec_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I, T_);
    return dk_check_launch("silu_mul");
  }
  const size_t total = (size_t)T_ * I;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == DK_F32)
    silu_mul_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)gu, (float*)out, I, total);
  else
    silu_mul_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I, total);
  return dk_check_launch("silu_mul");
}

// ------------------------------------------- rotary positions + cache append
// qkv[t] = [q (H*hd) | k (KV*hd) | v (KV*hd)].  For token t at position p of
// batch row b:
//   q and k are rotated with cos/sin of table[p] (pair j: angle p / theta^(2j/hd),
//   reference model.py:165-175); q stays in place, the rotated k and v go to page
//   block_table[b][p / ps], offset p % ps (reference eutils.py:36-66, model.py:474).
// Cache layout of one layer: [page][K|V][kv head][offset][hd].
// table == nullptr: no rotation (a mixer without rotary positions).
// kv == nullptr: the layer reads another layer's cache and appends nothing.
template <typename T>
__global__ void rope_append_kernel(T* __restrict__ qkv, const int* __restrict__ tok_pos, const int* __restrict__ tok_row,
                                   const int* __restrict__ block_table, int max_pages, T* __restrict__ kv, int num_pages,
                                   const float* __restrict__ table, int table_positions, int H, int KV, int hd, int ps,
                                   int interleaved, int* err) {
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int b = tok_row[t];
  const int half = hd / 2;
  const size_t stride = (size_t)(H + 2 * KV) * hd;
  T* base = qkv + (size_t)t * stride;
  if (pos < 0 || (table != nullptr && pos >= table_positions)) {
    if (threadIdx.x == 0) dk_report(err, DK_DEV_BAD_POSITION, t, pos, table_positions);
    return;
  }
  int page = -1;
  const int off = pos % ps;
  if (kv != nullptr) {
    const int lp = pos / ps;
    page = lp < max_pages ? block_table[(size_t)b * max_pages + lp] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) dk_report(err, DK_DEV_BAD_PAGE, t, lp, page);
      page = -1;
    }
  }
  const float* cs = table ? table + (size_t)pos * half * 2 : nullptr;
  for (int idx = threadIdx.x; idx < (H + KV) * half; idx += blockDim.x) {
    const int hs = idx / half, j = idx - hs * half;
    const int i0 = interleaved ? 2 * j : j;
    const int i1 = interleaved ? 2 * j + 1 : j + half;
    T* hp = base + (size_t)hs * hd;
    const float a = to_f32<T>(hp[i0]), bb = to_f32<T>(hp[i1]);
    float ra = a, rb = bb;
    if (cs) {
      const float c = cs[2 * j], s = cs[2 * j + 1];
      ra = a * c - bb * s;
      rb = a * s + bb * c;
    }
    const T ta = from_f32<T>(ra), tb = from_f32<T>(rb);
    hp[i0] = ta;
    hp[i1] = tb;
    if (hs >= H && page >= 0) {
      const int g = hs - H;
      T* dst = kv + ((((size_t)page * 2 + 0) * KV + g) * ps + off) * hd;
      dst[i0] = ta;
      dst[i1] = tb;
    }
  }
  if (page >= 0) {
    const T* vsrc = base + (size_t)(H + KV) * hd;
    for (int idx = threadIdx.x; idx < KV * hd; idx += blockDim.x) {
      const int g = idx / hd, dd = idx - g * hd;
      kv[((((size_t)page * 2 + 1) * KV + g) * ps + off) * hd + dd] = vsrc[idx];
    }
  }
}

// bfloat16, pairs (j, j + hd/2), head size a multiple of 16: eight pairs per thread with
// 16-byte loads and stores.
__global__ void rope_append_vec_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ tok_pos,
                                       const int* __restrict__ tok_row, const int* __restrict__ block_table, int max_pages,
                                       __nv_bfloat16* __restrict__ kv, int num_pages, const float* __restrict__ table,
                                       int table_positions, int H, int KV, int hd, int ps, int* err) {
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int b = tok_row[t];
  const int half = hd / 2, hv = half / 8;          // vectors per half head
  const size_t stride = (size_t)(H + 2 * KV) * hd;
  __nv_bfloat16* base = qkv + (size_t)t * stride;
  if (pos < 0 || (table != nullptr && pos >= table_positions)) {
    if (threadIdx.x == 0) dk_report(err, DK_DEV_BAD_POSITION, t, pos, table_positions);
    return;
  }
  int page = -1;
  const int off = pos % ps;
  if (kv != nullptr) {
    const int lp = pos / ps;
    page = lp < max_pages ? block_table[(size_t)b * max_pages + lp] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) dk_report(err, DK_DEV_BAD_PAGE, t, lp, page);
      page = -1;
    }
  }
  const float4* cs = table ? reinterpret_cast<const float4*>(table + (size_t)pos * half * 2) : nullptr;
  for (int idx = threadIdx.x; idx < (H + KV) * hv; idx += blockDim.x) {
    const int hs = idx / hv, jv = idx - hs * hv;
    __nv_bfloat16* hp = base + (size_t)hs * hd;
    uint4 av = *reinterpret_cast<const uint4*>(hp + jv * 8);
    uint4 bv = *reinterpret_cast<const uint4*>(hp + half + jv * 8);
    if (cs) {
      __nv_bfloat16* ae = reinterpret_cast<__nv_bfloat16*>(&av);
      __nv_bfloat16* be = reinterpret_cast<__nv_bfloat16*>(&bv);
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        const float4 c2 = cs[(jv * 8 + e) / 2];   // cos, sin of pair e and of pair e + 1
        const float a0 = __bfloat162float(ae[e]), b0 = __bfloat162float(be[e]);
        const float a1 = __bfloat162float(ae[e + 1]), b1 = __bfloat162float(be[e + 1]);
        ae[e] = __float2bfloat16_rn(a0 * c2.x - b0 * c2.y);
        be[e] = __float2bfloat16_rn(a0 * c2.y + b0 * c2.x);
        ae[e + 1] = __float2bfloat16_rn(a1 * c2.z - b1 * c2.w);
        be[e + 1] = __float2bfloat16_rn(a1 * c2.w + b1 * c2.z);
      }
      *reinterpret_cast<uint4*>(hp + jv * 8) = av;
      *reinterpret_cast<uint4*>(hp + half + jv * 8) = bv;
    }
    if (hs >= H && page >= 0) {
      __nv_bfloat16* dst = kv + ((((size_t)page * 2 + 0) * KV + (hs - H)) * ps + off) * hd;
      *reinterpret_cast<uint4*>(dst + jv * 8) = av;
      *reinterpret_cast<uint4*>(dst + half + jv * 8) = bv;
    }
  }
  if (page >= 0) {
    const __nv_bfloat16* vsrc = base + (size_t)(H + KV) * hd;
    const int vv = hd / 8;
    for (int idx = threadIdx.x; idx < KV * vv; idx += blockDim.x) {
      const int g = idx / vv, dv = idx - g * vv;
      *reinterpret_cast<uint4*>(kv + ((((size_t)page * 2 + 1) * KV + g) * ps + off) * hd + dv * 8) =
          *reinterpret_cast<const uint4*>(vsrc + (size_t)g * hd + dv * 8);
    }
  }
}

extern "C" int dk_rope_append(void* qkv, const int* tok_pos, const int* tok_row, const int* block_table, int max_pages,
                              void* kv, int num_pages, const float* table, int table_positions, int T_, int H, int KV,
                              int hd, int ps, int interleaved, int dtype, int* err, cudaStream_t stream) {
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && H > 0 && KV > 0 && hd > 0 && (hd % 2) == 0 && ps > 0,
             "rope_append: bad sizes T=%d H=%d KV=%d hd=%d ps=%d", T_, H, KV, hd, ps);
  DK_REQUIRE(kv == nullptr || (block_table != nullptr && max_pages > 0 && num_pages > 0),
             "rope_append: a cache is given without a block table");
  const int work = (H + KV) * hd / 2;
  const int threads = work >= 2048 ? 256 : 128;
  if (dtype == DK_BF16 && !interleaved && (hd % 16) == 0 && ((uintptr_t)qkv % 16) == 0 && ((uintptr_t)kv % 16) == 0) {
    const int vthreads = work / 8 >= 256 ? 256 : 128;
    rope_append_vec_kernel<<<T_, vthreads, 0, stream>>>((__nv_bfloat16*)qkv, tok_pos, tok_row, block_table, max_pages,
                                                        (__nv_bfloat16*)kv, num_pages, table, table_positions, H, KV, hd, ps, err);
    return dk_check_launch("rope_append");
  }
#define LAUNCH(T)                                                                                                   \
  rope_append_kernel<T><<<T_, threads, 0, stream>>>((T*)qkv, tok_pos, tok_row, block_table, max_pages, (T*)kv,      \
                                                     num_pages, table, table_positions, H, KV, hd, ps, interleaved, err)
  if (dtype == DK_F32) LAUNCH(float);
  else if (dtype == DK_BF16) LAUNCH(__nv_bfloat16);
  else DK_REQUIRE(false, "rope_append: unknown dtype %d", dtype);
#undef LAUNCH
  return dk_check_launch("rope_append");
}
