// Calibration statistics of the K/V rows a model writes into its cache, in one pass (sm_100a).
//
// The reference's capture hook (kvq/capture.py:25-44) keeps, per attention layer and per (kv head, channel), the
// running |x| maximum, signed maximum and minimum and a double-precision sum of K and of V, each as a separate
// torch reduction over the step's rows (eight passes over the data per layer and step). calib_stats_kernel reads
// every row once - 16-byte loads, rows whose slot is negative skipped like the hook's `slot_mapping >= 0` mask -
// and folds the step into the running statistics in place: maxima by integer atomics on the float bit patterns
// (exact and order-independent), sums carried per thread as unevaluated fp32 pairs (about 48 bits), folded over the
// block's token lanes and added to the fp64 totals with one atomicAdd per (block, channel).
#include <algorithm>

#include "kvq_common.cuh"

namespace kvq {
namespace {

constexpr int CS_THREADS = 256;

struct CalibArgs {
  const __nv_bfloat16 *key, *value;
  const int64_t* slots;   // may be null: every row counts
  float *k_absmax, *k_max, *k_min, *v_absmax, *v_max, *v_min;
  double *k_sum, *v_sum;
  long long* tokens;
  int64_t T, k_st, k_sh, v_st, v_sh;
  int H, D, groups;       // groups = H * D / 8 column groups of 8 channels
};

// max / min on floats stored as their bit patterns: non-negative floats order like ints, negative ones inversely
// like unsigned ints. The destination must hold a float (-inf / +inf / 0 to start with).
__device__ __forceinline__ void atomic_max_float(float* addr, float v) {
  if (v >= 0.f) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}
__device__ __forceinline__ void atomic_min_float(float* addr, float v) {
  if (v >= 0.f) atomicMin(reinterpret_cast<int*>(addr), __float_as_int(v));
  else atomicMax(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

struct Acc {
  float amax[8], mx[8], mn[8], hi[8], lo[8];
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int e = 0; e < 8; ++e) amax[e] = 0.f, mx[e] = -INFINITY, mn[e] = INFINITY, hi[e] = 0.f, lo[e] = 0.f;
  }
  __device__ __forceinline__ void add(const uint4& w) {
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float x = (e & 1) ? bf16hi(ww[e >> 1]) : bf16lo(ww[e >> 1]);
      amax[e] = fmaxf(amax[e], fabsf(x));
      mx[e] = fmaxf(mx[e], x);
      mn[e] = fminf(mn[e], x);
      // two-sum: hi + x = s + err exactly; the errors collect in lo
      const float s = __fadd_rn(hi[e], x);
      const float bb = __fadd_rn(s, -hi[e]);
      lo[e] = __fadd_rn(lo[e], __fadd_rn(__fadd_rn(hi[e], -__fadd_rn(s, -bb)), __fadd_rn(x, -bb)));
      hi[e] = s;
    }
  }
};

// Thread tid works on column group tid / lanes (8 channels) and token lane tid % lanes: the token lanes of a column
// group are neighbouring lanes of one warp, so a block folds them with shuffles and issues one set of atomics per
// (block, channel). Four rows are in flight per thread.
__global__ void __launch_bounds__(CS_THREADS) calib_stats_kernel(const CalibArgs a, int lanes) {
  __shared__ int s_rows;
  const int tid = threadIdx.x;
  const int cg = tid / lanes, tl = tid - cg * lanes;
  const bool active = cg < a.groups;
  const int h = (cg * 8) / a.D, c = (cg * 8) % a.D;
  if (tid == 0) s_rows = 0;
  __syncthreads();
  Acc k, v;
  k.init(), v.init();
  int rows = 0;
  if (active) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * lanes;
    for (int64_t t0 = static_cast<int64_t>(blockIdx.x) * lanes + tl; t0 < a.T; t0 += 4 * stride) {
      uint4 kw[4], vw[4];
      bool use[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int64_t t = t0 + i * stride;
        use[i] = t < a.T && !(a.slots && a.slots[t] < 0);
        if (use[i]) {
          kw[i] = ld_stream16(a.key + t * a.k_st + h * a.k_sh + c);
          vw[i] = ld_stream16(a.value + t * a.v_st + h * a.v_sh + c);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (use[i]) k.add(kw[i]), v.add(vw[i]), ++rows;
    }
  }
  // fold the token lanes of each column group (lanes is a power of two <= 32; all 32 lanes of a warp take part)
  const int o = h * a.D + c;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    double ks = static_cast<double>(k.hi[e]) + static_cast<double>(k.lo[e]);
    double vs = static_cast<double>(v.hi[e]) + static_cast<double>(v.lo[e]);
    for (int d = 1; d < lanes; d <<= 1) {
      k.amax[e] = fmaxf(k.amax[e], __shfl_xor_sync(0xffffffffu, k.amax[e], d));
      k.mx[e] = fmaxf(k.mx[e], __shfl_xor_sync(0xffffffffu, k.mx[e], d));
      k.mn[e] = fminf(k.mn[e], __shfl_xor_sync(0xffffffffu, k.mn[e], d));
      v.amax[e] = fmaxf(v.amax[e], __shfl_xor_sync(0xffffffffu, v.amax[e], d));
      v.mx[e] = fmaxf(v.mx[e], __shfl_xor_sync(0xffffffffu, v.mx[e], d));
      v.mn[e] = fminf(v.mn[e], __shfl_xor_sync(0xffffffffu, v.mn[e], d));
      ks += __shfl_xor_sync(0xffffffffu, ks, d);
      vs += __shfl_xor_sync(0xffffffffu, vs, d);
    }
    int any = rows;
    for (int d = 1; d < lanes; d <<= 1) any += __shfl_xor_sync(0xffffffffu, any, d);
    if (active && tl == 0 && any) {
      atomicMax(reinterpret_cast<int*>(a.k_absmax + o + e), __float_as_int(k.amax[e]));   // |x| >= 0
      atomicMax(reinterpret_cast<int*>(a.v_absmax + o + e), __float_as_int(v.amax[e]));
      atomic_max_float(a.k_max + o + e, k.mx[e] + 0.f);   // + 0: -0.0 becomes +0.0, whose bit pattern orders correctly
      atomic_min_float(a.k_min + o + e, k.mn[e] + 0.f);
      atomic_max_float(a.v_max + o + e, v.mx[e] + 0.f);
      atomic_min_float(a.v_min + o + e, v.mn[e] + 0.f);
      atomicAdd(a.k_sum + o + e, ks);
      atomicAdd(a.v_sum + o + e, vs);
    }
  }
  if (active && cg == 0 && rows) atomicAdd(&s_rows, rows);
  __syncthreads();
  if (tid == 0 && s_rows) atomicAdd(reinterpret_cast<unsigned long long*>(a.tokens), static_cast<unsigned long long>(s_rows));
}

}  // namespace
}  // namespace kvq

using namespace kvq;

extern "C" __attribute__((visibility("default"))) int kvq_calib_stats(
    const void* key, const void* value, const int64_t* slots, int64_t num_tokens, int num_kv_heads, int head_dim,
    int64_t key_stride_t, int64_t key_stride_h, int64_t value_stride_t, int64_t value_stride_h, float* k_absmax,
    float* k_max, float* k_min, double* k_sum, float* v_absmax, float* v_max, float* v_min, double* v_sum,
    long long* tokens, kvq_stream_t stream) {
  if (num_tokens <= 0) return KVQ_OK;
  KVQ_REQUIRE(key && value && k_absmax && k_max && k_min && k_sum && v_absmax && v_max && v_min && v_sum && tokens,
              "calib_stats: null pointer");
  KVQ_REQUIRE(num_kv_heads > 0 && head_dim > 0 && head_dim % 8 == 0, "calib_stats: head_dim must be a multiple of 8");
  const int groups = num_kv_heads * head_dim / 8;
  KVQ_REQUIRE(groups <= CS_THREADS, "calib_stats: at most %d channels per token (got %d)", CS_THREADS * 8,
              num_kv_heads * head_dim);
  KVQ_REQUIRE(aligned16(key) && aligned16(value) && key_stride_t % 8 == 0 && key_stride_h % 8 == 0 &&
                  value_stride_t % 8 == 0 && value_stride_h % 8 == 0,
              "calib_stats: rows must be 16-byte aligned");
  CalibArgs a;
  a.key = static_cast<const __nv_bfloat16*>(key), a.value = static_cast<const __nv_bfloat16*>(value), a.slots = slots;
  a.k_absmax = k_absmax, a.k_max = k_max, a.k_min = k_min, a.k_sum = k_sum;
  a.v_absmax = v_absmax, a.v_max = v_max, a.v_min = v_min, a.v_sum = v_sum, a.tokens = tokens;
  a.T = num_tokens, a.k_st = key_stride_t, a.k_sh = key_stride_h, a.v_st = value_stride_t, a.v_sh = value_stride_h;
  a.H = num_kv_heads, a.D = head_dim, a.groups = groups;
  int lanes = 1;   // token lanes per column group: the largest power of two that fits the block
  while (lanes * 2 * groups <= CS_THREADS && lanes < 32) lanes *= 2;
  int sms = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // one block per SM at most (every block ends with one set of atomics per channel), at least 4 rows per thread
  const int64_t blocks = std::max<int64_t>(1, std::min<int64_t>(sms, (num_tokens + lanes * 4 - 1) / (lanes * 4)));
  calib_stats_kernel<<<static_cast<unsigned>(blocks), CS_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a, lanes);
  KVQ_CUDA(cudaGetLastError());
  return KVQ_OK;
}
