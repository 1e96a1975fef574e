// Greedy and temperature sampling over float logits [R, V].
//
// Greedy: the highest logit, the lowest index among equals (reference:
// model.py:323).  Temperature: a draw from softmax(logits / T) (reference:
// eutils.py:103-111) by inverting the cumulative distribution in vocabulary
// order with one uniform number per draw.  The number comes from a counter-based
// generator, so a draw depends only on (seed of the request, position of the
// token), not on the batch or on how often a graph was replayed:
//   x = seed + (position + 1) * 0x9E3779B97F4A7C15
//   z = splitmix64 finaliser of x;  u = ((z >> 40) + 0.5) / 2^24
// top_p < 1 keeps the most probable tokens whose preceding mass is <= top_p
// (reference: eutils.py:81-101) and renormalises.
#include "common.cuh"

namespace {
constexpr int ST = 1024;

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  unsigned long long z = x;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}

__device__ __forceinline__ float uniform_of(unsigned long long seed, int position) {
  const unsigned long long x = seed + ((unsigned long long)position + 1ULL) * 0x9E3779B97F4A7C15ULL;
  const unsigned long long z = splitmix64(x);
  return ((float)(z >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

// argmax of a row with lowest-index tie break; every thread gets the result.
__device__ int block_argmax(const float* __restrict__ row, int V, float* s_val, int* s_idx, float* out_max) {
  float best = -INFINITY;
  int bi = 0x7fffffff;
  int i = threadIdx.x;
  // eight loads in flight per thread; indices grow within a thread, so ">" keeps the lowest index
  for (; i + 7 * (int)blockDim.x < V; i += 8 * blockDim.x) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = row[i + u * blockDim.x];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (v[u] > best) {
        best = v[u];
        bi = i + u * blockDim.x;
      }
  }
  for (; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v > best) {
      best = v;
      bi = i;
    }
  }
  if (bi == 0x7fffffff) bi = threadIdx.x < V ? threadIdx.x : 0;  // a row of NaN or -inf
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) {
    s_val[warp] = best;
    s_idx[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    best = lane < nw ? s_val[lane] : -INFINITY;
    bi = lane < nw ? s_idx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      s_val[32] = best;
      s_idx[32] = bi;
    }
  }
  __syncthreads();
  if (out_max) *out_max = s_val[32];
  return s_idx[32];
}

__global__ void __launch_bounds__(ST) sample_kernel(const float* __restrict__ logits, int ldl, int V,
                                                    const float* __restrict__ temperature, const float* __restrict__ top_p,
                                                    const unsigned long long* __restrict__ seeds,
                                                    const int* __restrict__ positions, int* __restrict__ out,
                                                    const int* __restrict__ status) {
  __shared__ float s_val[33];
  __shared__ int s_idx[33];
  __shared__ float s_scan[ST];
  __shared__ float s_red[34];
  __shared__ int s_pick;
  const int r = blockIdx.x;
  // the kernels' error record as it stands when the step's last kernel runs, behind the tokens
  if (status != nullptr && r == 0 && threadIdx.x < 4) out[gridDim.x + threadIdx.x] = status[threadIdx.x];
  const float* row = logits + (size_t)r * ldl;
  const float temp = temperature ? temperature[r] : 0.f;
  float mx;
  const int amax = block_argmax(row, V, s_val, s_idx, &mx);
  if (!(temp > 0.f)) {
    if (threadIdx.x == 0) {
      out[r] = amax;
    }
    return;
  }
  const float inv_t = 1.f / temp;
  // weight of token i: e_i = exp((l_i - max) / T); the top-p filter keeps i when
  // the mass of the strictly more probable tokens is <= top_p * Z.
  float cut = -INFINITY;  // keep tokens with logit >= cut
  const float tp = top_p ? top_p[r] : 1.f;
  float z = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) z += expf((row[i] - mx) * inv_t);
  z = block_sum(z, s_red);
  if (tp < 1.f) {
    // bisection on the logit value: mass_above(c) = sum of e_i with l_i > c is
    // non-increasing in c; the smallest kept logit is the lowest c with
    // mass_above(c) <= top_p * Z among the row's own values.
    float lo_c = -INFINITY, hi_c = mx;  // mass_above(hi_c) = 0 <= target always
    float lo_f = mx - 80.f * temp;      // below this e_i underflows to nothing that matters
    lo_c = lo_f;
    for (int it = 0; it < 32; ++it) {
      const float mid = 0.5f * (lo_c + hi_c);
      float ma = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float l = row[i];
        if (l > mid) ma += expf((l - mx) * inv_t);
      }
      ma = block_sum(ma, s_red);
      if (ma <= tp * z) hi_c = mid; else lo_c = mid;
    }
    // hi_c: mass strictly above it is within top_p, so every token with
    // l >= (smallest row value > lo_c) is kept; take the lowest row value above lo_c.
    float near = INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float l = row[i];
      if (l > lo_c && l < near) near = l;
    }
    near = -block_max(-near, s_red);
    cut = near;
    z = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float l = row[i];
      if (l >= cut) z += expf((l - mx) * inv_t);
    }
    z = block_sum(z, s_red);
  }
  const float u = uniform_of(seeds ? seeds[r] : 0ULL, positions ? positions[r] : 0);
  const float target = u * z;
  // each thread owns a contiguous segment of the vocabulary
  const int seg = (V + ST - 1) / ST;
  const int b0 = threadIdx.x * seg;
  const int b1 = b0 + seg < V ? b0 + seg : V;
  float mine = 0.f;
  for (int i = b0; i < b1; ++i) {
    const float l = row[i];
    if (l >= cut) mine += expf((l - mx) * inv_t);
  }
  s_scan[threadIdx.x] = mine;
  if (threadIdx.x == 0) s_pick = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.f;
    int owner = -1;
    for (int i = 0; i < ST; ++i) {
      const float nxt = run + s_scan[i];
      if (owner < 0 && s_scan[i] > 0.f && target < nxt) {
        owner = i;
        s_red[33] = run;
      }
      run = nxt;
    }
    if (owner < 0) {  // rounding left the target at or past the end: last segment with mass
      run = 0.f;
      for (int i = 0; i < ST; ++i) {
        if (s_scan[i] > 0.f) {
          owner = i;
          s_red[33] = run;
        }
        run += s_scan[i];
      }
    }
    s_idx[0] = owner;
  }
  __syncthreads();
  if (threadIdx.x == s_idx[0]) {
    float run = s_red[33];
    int pick = -1, last = -1;
    for (int i = b0; i < b1; ++i) {
      const float l = row[i];
      if (l >= cut) {
        run += expf((l - mx) * inv_t);
        last = i;
        if (target < run) {
          pick = i;
          break;
        }
      }
    }
    if (pick < 0) pick = last >= 0 ? last : amax;
    out[r] = pick;

  }
}
}  // namespace

extern "C" int dk_sample(const float* logits, int ldl, int R, int V, const float* temperature, const float* top_p,
                         const unsigned long long* seeds, const int* positions, int* out, const int* status,
                         cudaStream_t stream) {
  if (R == 0) return 0;
  DK_REQUIRE(R > 0 && V > 0 && ldl >= V, "sample: bad sizes R=%d V=%d ld=%d", R, V, ldl);
  sample_kernel<<<R, ST, 0, stream>>>(logits, ldl, V, temperature, top_p, seeds, positions, out, status);
  return dk_check_launch("sample");
}
