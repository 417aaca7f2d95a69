// Elementwise kernels of the static INT8 KV-cache path: fused quantize + paged cache write, standalone q
// quantization, page dequantization. All three are pure HBM streaming work: one thread moves 16 channels
// with 16-byte loads and 16-byte stores, and the grid is flat over (row, 16-channel group) items.
#include "kvq_common.cuh"

namespace kvq {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ void load16f(const float* p, float (&x)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(p) + i);
    x[4 * i] = v.x, x[4 * i + 1] = v.y, x[4 * i + 2] = v.z, x[4 * i + 3] = v.w;
  }
}

__device__ __forceinline__ void load16bf(const __nv_bfloat16* p, float (&x)[16]) {
  const uint4 a = ld_stream16(p), b = ld_stream16(p + 8);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) x[2 * i] = bf16lo(w[i]), x[2 * i + 1] = bf16hi(w[i]);
}

// ------------------------------------------------------------------------------------------------------
// Fused quantize + cache write. Item = (token, kv head, 16-channel group).
// ------------------------------------------------------------------------------------------------------
struct QuantCacheArgs {
  const __nv_bfloat16 *key, *value;
  int8_t *kc, *vc;
  const int64_t* slots;
  const float *ks, *vs, *kmu;
  int64_t n_items;
  int H, D, groups;  // groups = D / 16
  int block_size, bs_shift;  // bs_shift >= 0 when block_size is a power of two
  int64_t k_st, k_sh, v_st, v_sh, kc_sb, kc_sn, kc_sh, vc_sb, vc_sn, vc_sh;
  int pc_k, pc_v;
};

__global__ void __launch_bounds__(kThreads) quant_cache_kernel(const QuantCacheArgs a) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (i >= a.n_items) return;
  const int per_tok = a.H * a.groups;
  const int64_t tok = i / per_tok;
  const int rem = static_cast<int>(i - tok * per_tok);
  const int h = rem / a.groups, d0 = (rem - h * a.groups) * 16;
  // every load below is independent of the slot: issue them all before looking at it (one DRAM round trip)
  float k[16], v[16], sk[16], sv[16], mu[16];
  load16bf(a.key + tok * a.k_st + h * a.k_sh + d0, k);
  load16bf(a.value + tok * a.v_st + h * a.v_sh + d0, v);
  const int64_t slot = __ldg(a.slots + tok);
  load16f(a.kmu + h * a.D + d0, mu);
  if (a.pc_k) {
    load16f(a.ks + h * a.D + d0, sk);
  } else {
    const float s = __ldg(a.ks + h);
#pragma unroll
    for (int e = 0; e < 16; ++e) sk[e] = s;
  }
  if (a.pc_v) {
    load16f(a.vs + h * a.D + d0, sv);
  } else {
    const float s = __ldg(a.vs + h);
#pragma unroll
    for (int e = 0; e < 16; ++e) sv[e] = s;
  }
  if (slot < 0) return;  // padding token
  int64_t blk, off;
  if (a.bs_shift >= 0) {
    blk = slot >> a.bs_shift, off = slot & (a.block_size - 1);
  } else {
    blk = slot / a.block_size, off = slot - blk * a.block_size;
  }
  uint32_t kw[4], vw[4];
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    // fp32 subtract, IEEE divide, round half to even, clamp: the order the torch quantizer uses
    kw[w] = pack4(quant1(__fsub_rn(k[4 * w], mu[4 * w]), sk[4 * w]), quant1(__fsub_rn(k[4 * w + 1], mu[4 * w + 1]), sk[4 * w + 1]),
                  quant1(__fsub_rn(k[4 * w + 2], mu[4 * w + 2]), sk[4 * w + 2]),
                  quant1(__fsub_rn(k[4 * w + 3], mu[4 * w + 3]), sk[4 * w + 3]));
    vw[w] = pack4(quant1(v[4 * w], sv[4 * w]), quant1(v[4 * w + 1], sv[4 * w + 1]), quant1(v[4 * w + 2], sv[4 * w + 2]),
                  quant1(v[4 * w + 3], sv[4 * w + 3]));
  }
  *reinterpret_cast<uint4*>(a.kc + blk * a.kc_sb + off * a.kc_sn + h * a.kc_sh + d0) = make_uint4(kw[0], kw[1], kw[2], kw[3]);
  *reinterpret_cast<uint4*>(a.vc + blk * a.vc_sb + off * a.vc_sn + h * a.vc_sh + d0) = make_uint4(vw[0], vw[1], vw[2], vw[3]);
}

// ------------------------------------------------------------------------------------------------------
// q fold + quantize. 8 lanes per (token, q head) row of 128 channels, 16 channels per lane.
// ------------------------------------------------------------------------------------------------------
template <int GROUP>
__global__ void __launch_bounds__(kThreads) quant_q_kernel(const __nv_bfloat16* __restrict__ q, const float* __restrict__ ks,
                                                           int8_t* __restrict__ q_i8, float* __restrict__ q_scale,
                                                           int64_t n_rows, int Hq, int G, int64_t q_st, int64_t q_sh,
                                                           int pc_k) {
  constexpr int D = 128, LPR = D / 16;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  const int part = static_cast<int>(i % LPR);
  const int64_t row = i / LPR;
  const bool live = row < n_rows;
  const int64_t r = live ? row : n_rows - 1;  // idle lanes of the last warp still take part in the shuffles
  const int64_t t = r / Hq;
  const int h = static_cast<int>(r - t * Hq), d0 = part * 16;
  float x[16];
  load16bf(q + t * q_st + h * q_sh + d0, x);
  if (pc_k) {
    float s[16];
    load16f(ks + (h / G) * D + d0, s);
#pragma unroll
    for (int e = 0; e < 16; ++e) x[e] = __fmul_rn(x[e], s[e]);
  }
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < 16; ++e) amax = fmaxf(amax, fabsf(x[e]));
#pragma unroll
  for (int o = 1; o < GROUP / 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = fmaxf(__fdiv_rn(amax, 127.f), 1e-8f);
  if (!live) return;
  uint32_t w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k)
    w[k] = pack4(quant1(x[4 * k], s), quant1(x[4 * k + 1], s), quant1(x[4 * k + 2], s), quant1(x[4 * k + 3], s));
  *reinterpret_cast<uint4*>(q_i8 + row * D + d0) = make_uint4(w[0], w[1], w[2], w[3]);
  if (part % (GROUP / 16) == 0) q_scale[row * (D / GROUP) + d0 / GROUP] = s;
}

// ------------------------------------------------------------------------------------------------------
// Page dequantization. Item = (output page, slot, kv head, 16-channel group); the output is contiguous
// [pages, block, H, D], so item i of page p writes 32 bytes at element offset 16 * (p * items_per_page + i).
// ------------------------------------------------------------------------------------------------------
struct DequantArgs {
  const int8_t *kc, *vc;
  __nv_bfloat16 *ko, *vo;
  const int32_t *block_table, *src_req, *src_j;
  const float *ks, *vs;
  int64_t n_items, bt_stride;
  int H, D, groups, block_size;
  int64_t kc_sb, kc_sn, kc_sh, vc_sb, vc_sn, vc_sh;
  int pc_k, pc_v;
};

__device__ __forceinline__ void dequant_store(uint4 raw, __nv_bfloat16* dst, const float* scale, int per_channel) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  float s[16];
  if (per_channel) {
    load16f(scale, s);
  } else {
    const float one = __ldg(scale);
#pragma unroll
    for (int e = 0; e < 16; ++e) s[e] = one;
  }
  uint32_t o[8];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    // int8 -> fp32 (exact), fp32 multiply, round to nearest even bf16
    const float f0 = static_cast<float>(static_cast<int8_t>(w[k] & 0xff));
    const float f1 = static_cast<float>(static_cast<int8_t>((w[k] >> 8) & 0xff));
    const float f2 = static_cast<float>(static_cast<int8_t>((w[k] >> 16) & 0xff));
    const float f3 = static_cast<float>(static_cast<int8_t>(w[k] >> 24));
    o[2 * k] = pack_bf16x2(__fmul_rn(f0, s[4 * k]), __fmul_rn(f1, s[4 * k + 1]));
    o[2 * k + 1] = pack_bf16x2(__fmul_rn(f2, s[4 * k + 2]), __fmul_rn(f3, s[4 * k + 3]));
  }
  reinterpret_cast<uint4*>(dst)[0] = make_uint4(o[0], o[1], o[2], o[3]);
  reinterpret_cast<uint4*>(dst)[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// One CTA per output page: the source page id is looked up once, then every thread issues all of its 16-byte
// loads (kUnroll items of K and of V) before converting any of them.
constexpr int kUnroll = 2;

__global__ void __launch_bounds__(kThreads) dequant_pages_kernel(const DequantArgs a) {
  const int64_t p = blockIdx.x;
  const int per_slot = a.H * a.groups, per_page = a.block_size * per_slot;
  const int64_t src = __ldg(a.block_table + static_cast<int64_t>(__ldg(a.src_req + p)) * a.bt_stride + __ldg(a.src_j + p));
  const int8_t* kp = a.kc + src * a.kc_sb;
  const int8_t* vp = a.vc + src * a.vc_sb;
  for (int base = threadIdx.x; base < per_page; base += kThreads * kUnroll) {
    uint4 kr[kUnroll], vr[kUnroll];
    int hh[kUnroll], dd[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int i = base + u * kThreads;
      const int n = i / per_slot, rem = i - n * per_slot;
      hh[u] = rem / a.groups, dd[u] = (rem - hh[u] * a.groups) * 16;
      if (i < per_page) {
        kr[u] = ld_stream16(kp + n * a.kc_sn + hh[u] * a.kc_sh + dd[u]);
        vr[u] = ld_stream16(vp + n * a.vc_sn + hh[u] * a.vc_sh + dd[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int i = base + u * kThreads;
      if (i >= per_page) continue;
      const int64_t o = (p * per_page + i) * 16;
      dequant_store(kr[u], a.ko + o, a.pc_k ? a.ks + hh[u] * a.D + dd[u] : a.ks + hh[u], a.pc_k);
      dequant_store(vr[u], a.vo + o, a.pc_v ? a.vs + hh[u] * a.D + dd[u] : a.vs + hh[u], a.pc_v);
    }
  }
}

int ilog2_exact(int x) {
  if (x <= 0 || (x & (x - 1))) return -1;
  int s = 0;
  while ((1 << s) < x) ++s;
  return s;
}

}  // namespace
}  // namespace kvq

using namespace kvq;

extern "C" __attribute__((visibility("default"))) int kvq_quant_cache(const void* key, const void* value, void* k_cache, void* v_cache, const int64_t* slots,
                               const float* k_scale, const float* v_scale, const float* k_mu, int64_t num_tokens,
                               int num_kv_heads, int head_dim, int block_size, int64_t key_stride_t,
                               int64_t key_stride_h, int64_t value_stride_t, int64_t value_stride_h,
                               int64_t kc_stride_b, int64_t kc_stride_n, int64_t kc_stride_h, int64_t vc_stride_b,
                               int64_t vc_stride_n, int64_t vc_stride_h, int k_per_channel, int v_per_channel,
                               kvq_stream_t stream) {
  KVQ_REQUIRE(head_dim == 64 || head_dim == 128, "head_dim must be 64 or 128, got %d", head_dim);
  KVQ_REQUIRE(num_tokens >= 0 && num_kv_heads > 0 && block_size > 0, "quant_cache: bad sizes");
  if (num_tokens == 0) return KVQ_OK;
  KVQ_REQUIRE(key && value && k_cache && v_cache && slots && k_scale && v_scale && k_mu, "quant_cache: null pointer");
  KVQ_REQUIRE(aligned16(key) && aligned16(value) && key_stride_t % 8 == 0 && key_stride_h % 8 == 0 &&
                  value_stride_t % 8 == 0 && value_stride_h % 8 == 0,
              "quant_cache: key/value rows must be 16-byte aligned");
  KVQ_REQUIRE(aligned16(k_cache) && aligned16(v_cache) && kc_stride_b % 16 == 0 && kc_stride_n % 16 == 0 &&
                  kc_stride_h % 16 == 0 && vc_stride_b % 16 == 0 && vc_stride_n % 16 == 0 && vc_stride_h % 16 == 0,
              "quant_cache: cache rows must be 16-byte aligned");
  KVQ_REQUIRE(aligned16(k_scale) && aligned16(v_scale) && aligned16(k_mu), "quant_cache: scales must be 16-byte aligned");
  QuantCacheArgs a;
  a.key = static_cast<const __nv_bfloat16*>(key), a.value = static_cast<const __nv_bfloat16*>(value);
  a.kc = static_cast<int8_t*>(k_cache), a.vc = static_cast<int8_t*>(v_cache);
  a.slots = slots, a.ks = k_scale, a.vs = v_scale, a.kmu = k_mu;
  a.H = num_kv_heads, a.D = head_dim, a.groups = head_dim / 16;
  a.n_items = num_tokens * num_kv_heads * a.groups;
  a.block_size = block_size, a.bs_shift = ilog2_exact(block_size);
  a.k_st = key_stride_t, a.k_sh = key_stride_h, a.v_st = value_stride_t, a.v_sh = value_stride_h;
  a.kc_sb = kc_stride_b, a.kc_sn = kc_stride_n, a.kc_sh = kc_stride_h;
  a.vc_sb = vc_stride_b, a.vc_sn = vc_stride_n, a.vc_sh = vc_stride_h;
  a.pc_k = k_per_channel, a.pc_v = v_per_channel;
  const int64_t blocks = (a.n_items + kThreads - 1) / kThreads;
  quant_cache_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  KVQ_CUDA(cudaGetLastError());
  return KVQ_OK;
}

extern "C" __attribute__((visibility("default"))) int kvq_quant_q(const void* q, const float* k_scale, void* q_i8, float* q_scale, int64_t num_tokens,
                           int num_q_heads, int num_kv_heads, int head_dim, int group, int64_t q_stride_t,
                           int64_t q_stride_h, int k_per_channel, kvq_stream_t stream) {
  KVQ_REQUIRE(head_dim == 128 && (group == 128 || group == 32), "standalone q quantization: head_dim 128, group 128 or 32");
  KVQ_REQUIRE(num_q_heads > 0 && num_kv_heads > 0 && num_q_heads % num_kv_heads == 0, "quant_q: bad head counts");
  if (num_tokens <= 0) return KVQ_OK;
  KVQ_REQUIRE(q && q_i8 && q_scale && (k_scale || !k_per_channel), "quant_q: null pointer");
  KVQ_REQUIRE(aligned16(q) && q_stride_t % 8 == 0 && q_stride_h % 8 == 0 && aligned16(q_i8) &&
                  (!k_per_channel || aligned16(k_scale)),
              "quant_q: rows must be 16-byte aligned");
  const int64_t rows = num_tokens * num_q_heads;
  const int64_t blocks = (rows * 8 + kThreads - 1) / kThreads;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  const auto* qp = static_cast<const __nv_bfloat16*>(q);
  auto* qi = static_cast<int8_t*>(q_i8);
  const int G = num_q_heads / num_kv_heads;
  if (group == 128)
    quant_q_kernel<128><<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(qp, k_scale, qi, q_scale, rows, num_q_heads, G,
                                                                           q_stride_t, q_stride_h, k_per_channel);
  else
    quant_q_kernel<32><<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(qp, k_scale, qi, q_scale, rows, num_q_heads, G,
                                                                          q_stride_t, q_stride_h, k_per_channel);
  KVQ_CUDA(cudaGetLastError());
  return KVQ_OK;
}

extern "C" __attribute__((visibility("default"))) int kvq_dequant_pages(const void* k_cache, const void* v_cache, void* k_out, void* v_out,
                                 const int32_t* block_table, const int32_t* src_req, const int32_t* src_j,
                                 const float* k_scale, const float* v_scale, int64_t num_pages, int num_kv_heads,
                                 int head_dim, int block_size, int64_t kc_stride_b, int64_t kc_stride_n,
                                 int64_t kc_stride_h, int64_t vc_stride_b, int64_t vc_stride_n, int64_t vc_stride_h,
                                 int64_t bt_stride, int k_per_channel, int v_per_channel, kvq_stream_t stream) {
  KVQ_REQUIRE(head_dim == 64 || head_dim == 128, "head_dim must be 64 or 128, got %d", head_dim);
  KVQ_REQUIRE(num_kv_heads > 0 && block_size > 0, "dequant_pages: bad sizes");
  if (num_pages <= 0) return KVQ_OK;
  KVQ_REQUIRE(k_cache && v_cache && k_out && v_out && block_table && src_req && src_j && k_scale && v_scale,
              "dequant_pages: null pointer");
  KVQ_REQUIRE(aligned16(k_cache) && aligned16(v_cache) && aligned16(k_out) && aligned16(v_out) && kc_stride_b % 16 == 0 &&
                  kc_stride_n % 16 == 0 && kc_stride_h % 16 == 0 && vc_stride_b % 16 == 0 && vc_stride_n % 16 == 0 &&
                  vc_stride_h % 16 == 0,
              "dequant_pages: rows must be 16-byte aligned");
  DequantArgs a;
  a.kc = static_cast<const int8_t*>(k_cache), a.vc = static_cast<const int8_t*>(v_cache);
  a.ko = static_cast<__nv_bfloat16*>(k_out), a.vo = static_cast<__nv_bfloat16*>(v_out);
  a.block_table = block_table, a.src_req = src_req, a.src_j = src_j, a.ks = k_scale, a.vs = v_scale;
  a.H = num_kv_heads, a.D = head_dim, a.groups = head_dim / 16, a.block_size = block_size;
  a.n_items = num_pages * block_size * num_kv_heads * a.groups;
  a.bt_stride = bt_stride;
  a.kc_sb = kc_stride_b, a.kc_sn = kc_stride_n, a.kc_sh = kc_stride_h;
  a.vc_sb = vc_stride_b, a.vc_sn = vc_stride_n, a.vc_sh = vc_stride_h;
  a.pc_k = k_per_channel, a.pc_v = v_per_channel;
  dequant_pages_kernel<<<static_cast<unsigned>(num_pages), kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  KVQ_CUDA(cudaGetLastError());
  return KVQ_OK;
}
