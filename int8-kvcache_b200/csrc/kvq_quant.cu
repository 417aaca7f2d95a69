// Elementwise kernels of the static INT8 KV-cache path: fused quantize + paged cache write, standalone q
// quantization, page dequantization. All three are pure HBM streaming work. The write and dequantize kernels
// move 8 channels per item, so that both sides are fully coalesced: 16-byte loads of bf16 / 8-byte stores of
// int8 when quantizing, 8-byte loads / 16-byte stores when dequantizing (consecutive lanes touch consecutive
// bytes in every instruction); each thread has several items in flight.
#include "kvq_common.cuh"

namespace kvq {
namespace {

constexpr int kThreads = 256;

// 8 scale values for channels d0..d0+7 of head h: per channel from [H, D], or the head's single value.
__device__ __forceinline__ void load_scale8(const float* base, int per_channel, int h, int D, int d0, float (&s)[8]) {
  if (per_channel) {
    const float4 lo = __ldg(reinterpret_cast<const float4*>(base + h * D + d0));
    const float4 hi = __ldg(reinterpret_cast<const float4*>(base + h * D + d0) + 1);
    s[0] = lo.x, s[1] = lo.y, s[2] = lo.z, s[3] = lo.w, s[4] = hi.x, s[5] = hi.y, s[6] = hi.z, s[7] = hi.w;
  } else {
    const float one = __ldg(base + h);
#pragma unroll
    for (int e = 0; e < 8; ++e) s[e] = one;
  }
}

__device__ __forceinline__ uint2 ld_stream8(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

// ------------------------------------------------------------------------------------------------------
// Fused quantize + cache write. Item = (token, kv head, 8-channel group); kItems items per thread, one block of
// kThreads * kItems consecutive items per CTA, every load issued before the first use.
// ------------------------------------------------------------------------------------------------------
struct QuantCacheArgs {
  const __nv_bfloat16 *key, *value;
  int8_t *kc, *vc;
  const int64_t* slots;
  const float *ks, *vs, *kmu;
  int64_t n_items;
  int H, D, groups;  // groups = D / 8
  int block_size, bs_shift;  // bs_shift >= 0 when block_size is a power of two
  int64_t k_st, k_sh, v_st, v_sh, kc_sb, kc_sn, kc_sh, vc_sb, vc_sn, vc_sh;
  int pc_k, pc_v;
};

constexpr int kItems = 2;

__device__ __forceinline__ uint2 quant8(uint4 raw, const float (&mu)[8], const float (&sc)[8], bool centre) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  int q[8];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    // fp32 subtract, IEEE divide, round half to even, clamp: the order the torch quantizer uses
    const float lo = bf16lo(w[k]), hi = bf16hi(w[k]);
    q[2 * k] = quant1(centre ? __fsub_rn(lo, mu[2 * k]) : lo, sc[2 * k]);
    q[2 * k + 1] = quant1(centre ? __fsub_rn(hi, mu[2 * k + 1]) : hi, sc[2 * k + 1]);
  }
  return make_uint2(pack4(q[0], q[1], q[2], q[3]), pack4(q[4], q[5], q[6], q[7]));
}

__global__ void __launch_bounds__(kThreads) quant_cache_kernel(const QuantCacheArgs a) {
  const int per_tok = a.H * a.groups;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * (kThreads * kItems) + threadIdx.x;
  uint4 kr[kItems], vr[kItems];
  int64_t slot[kItems];
  int hh[kItems], dd[kItems];
#pragma unroll
  for (int u = 0; u < kItems; ++u) {
    const int64_t i = base + u * kThreads;
    slot[u] = -1;
    if (i < a.n_items) {
      const int64_t tok = i / per_tok;
      const int rem = static_cast<int>(i - tok * per_tok);
      hh[u] = rem / a.groups, dd[u] = (rem - hh[u] * a.groups) * 8;
      kr[u] = ld_stream16(a.key + tok * a.k_st + hh[u] * a.k_sh + dd[u]);
      vr[u] = ld_stream16(a.value + tok * a.v_st + hh[u] * a.v_sh + dd[u]);
      slot[u] = __ldg(a.slots + tok);
    }
  }
#pragma unroll
  for (int u = 0; u < kItems; ++u) {
    if (slot[u] < 0) continue;  // padding token (or past the end)
    int64_t blk, off;
    if (a.bs_shift >= 0) {
      blk = slot[u] >> a.bs_shift, off = slot[u] & (a.block_size - 1);
    } else {
      blk = slot[u] / a.block_size, off = slot[u] - blk * a.block_size;
    }
    float sk[8], sv[8], mu[8];
    load_scale8(a.kmu, 1, hh[u], a.D, dd[u], mu);
    load_scale8(a.ks, a.pc_k, hh[u], a.D, dd[u], sk);
    load_scale8(a.vs, a.pc_v, hh[u], a.D, dd[u], sv);
    *reinterpret_cast<uint2*>(a.kc + blk * a.kc_sb + off * a.kc_sn + hh[u] * a.kc_sh + dd[u]) = quant8(kr[u], mu, sk, true);
    *reinterpret_cast<uint2*>(a.vc + blk * a.vc_sb + off * a.vc_sn + hh[u] * a.vc_sh + dd[u]) = quant8(vr[u], mu, sv, false);
  }
}

// ------------------------------------------------------------------------------------------------------
// q fold + quantize. 16 lanes per (token, q head) row of 128 channels, 8 channels per lane: one 16-byte load,
// one 8-byte store, abs-max over the 16 (group 128) or 4 (group 32) lanes of a group by shuffles.
// ------------------------------------------------------------------------------------------------------
template <int GROUP>
__global__ void __launch_bounds__(kThreads) quant_q_kernel(const __nv_bfloat16* __restrict__ q, const float* __restrict__ ks,
                                                           int8_t* __restrict__ q_i8, float* __restrict__ q_scale,
                                                           int64_t n_rows, int Hq, int G, int64_t q_st, int64_t q_sh,
                                                           int pc_k) {
  constexpr int D = 128, LPR = D / 8;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  const int part = static_cast<int>(i % LPR);
  const int64_t row = i / LPR;
  const bool live = row < n_rows;
  const int64_t r = live ? row : n_rows - 1;  // idle lanes of the last warp still take part in the shuffles
  const int64_t t = r / Hq;
  const int h = static_cast<int>(r - t * Hq), d0 = part * 8;
  const uint4 raw = ld_stream16(q + t * q_st + h * q_sh + d0);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  float x[8];
#pragma unroll
  for (int k = 0; k < 4; ++k) x[2 * k] = bf16lo(w[k]), x[2 * k + 1] = bf16hi(w[k]);
  if (pc_k) {   // a per-head K scale is not folded into q and k_scale is not read
    float s8[8];
    load_scale8(ks, 1, h / G, D, d0, s8);
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] = __fmul_rn(x[e], s8[e]);
  }
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(x[e]));
#pragma unroll
  for (int o = 1; o < GROUP / 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = fmaxf(__fdiv_rn(amax, 127.f), 1e-8f);
  if (!live) return;
  *reinterpret_cast<uint2*>(q_i8 + row * D + d0) =
      make_uint2(pack4(quant1(x[0], s), quant1(x[1], s), quant1(x[2], s), quant1(x[3], s)),
                 pack4(quant1(x[4], s), quant1(x[5], s), quant1(x[6], s), quant1(x[7], s)));
  if (part % (GROUP / 8) == 0) q_scale[row * (D / GROUP) + d0 / GROUP] = s;
}

// ------------------------------------------------------------------------------------------------------
// Page dequantization. Item = (output page, slot, kv head, 8-channel group); the output is contiguous
// [pages, block, H, D], so item i of page p writes 16 bytes at element offset 8 * (p * items_per_page + i).
// One CTA per output page: the source page id is looked up once, then every thread issues all of its 8-byte
// loads (kDqItems items of K and of V) before converting any of them.
// ------------------------------------------------------------------------------------------------------
struct DequantArgs {
  const int8_t *kc, *vc;
  __nv_bfloat16 *ko, *vo;
  const int32_t *block_table, *src_req, *src_j;
  const float *ks, *vs;
  int64_t bt_stride;
  int H, D, groups, block_size;   // groups = D / 8
  int64_t kc_sb, kc_sn, kc_sh, vc_sb, vc_sn, vc_sh;
  int pc_k, pc_v;
};

constexpr int kDqItems = 4;

__device__ __forceinline__ uint4 dequant8(uint2 raw, const float (&s)[8]) {
  const uint32_t w[2] = {raw.x, raw.y};
  uint32_t o[4];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    // int8 -> fp32 (exact), fp32 multiply, round to nearest even bf16
    const float f0 = static_cast<float>(static_cast<int8_t>(w[k] & 0xff));
    const float f1 = static_cast<float>(static_cast<int8_t>((w[k] >> 8) & 0xff));
    const float f2 = static_cast<float>(static_cast<int8_t>((w[k] >> 16) & 0xff));
    const float f3 = static_cast<float>(static_cast<int8_t>(w[k] >> 24));
    o[2 * k] = pack_bf16x2(__fmul_rn(f0, s[4 * k]), __fmul_rn(f1, s[4 * k + 1]));
    o[2 * k + 1] = pack_bf16x2(__fmul_rn(f2, s[4 * k + 2]), __fmul_rn(f3, s[4 * k + 3]));
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

__global__ void __launch_bounds__(kThreads) dequant_pages_kernel(const DequantArgs a) {
  const int64_t p = blockIdx.x;
  const int per_slot = a.H * a.groups, per_page = a.block_size * per_slot;
  const int64_t src = __ldg(a.block_table + static_cast<int64_t>(__ldg(a.src_req + p)) * a.bt_stride + __ldg(a.src_j + p));
  const int8_t* kp = a.kc + src * a.kc_sb;
  const int8_t* vp = a.vc + src * a.vc_sb;
  for (int base = threadIdx.x; base < per_page; base += kThreads * kDqItems) {
    uint2 kr[kDqItems], vr[kDqItems];
    int hh[kDqItems], dd[kDqItems];
#pragma unroll
    for (int u = 0; u < kDqItems; ++u) {
      const int i = base + u * kThreads;
      const int n = i / per_slot, rem = i - n * per_slot;
      hh[u] = rem / a.groups, dd[u] = (rem - hh[u] * a.groups) * 8;
      if (i < per_page) {
        kr[u] = ld_stream8(kp + n * a.kc_sn + hh[u] * a.kc_sh + dd[u]);
        vr[u] = ld_stream8(vp + n * a.vc_sn + hh[u] * a.vc_sh + dd[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < kDqItems; ++u) {
      const int i = base + u * kThreads;
      if (i >= per_page) continue;
      const int64_t o = (p * per_page + i) * 8;
      float sk[8], sv[8];
      load_scale8(a.ks, a.pc_k, hh[u], a.D, dd[u], sk);
      load_scale8(a.vs, a.pc_v, hh[u], a.D, dd[u], sv);
      *reinterpret_cast<uint4*>(a.ko + o) = dequant8(kr[u], sk);
      *reinterpret_cast<uint4*>(a.vo + o) = dequant8(vr[u], sv);
    }
  }
}

// ------------------------------------------------------------------------------------------------------
// Raw int8 pages to and from a contiguous wire buffer (prefill / decode disaggregation). Wire page p holds cache
// page page_ids[p] as [K | V][block][H][D] bytes; one CTA per page, 16 bytes per item, every load of a thread issued
// before its first store. Static scales are not part of the transfer: both sides load the same scale file.
// ------------------------------------------------------------------------------------------------------
struct WireArgs {
  int8_t *kc, *vc;          // cache views (read when exporting, written when importing)
  int8_t* wire;             // [pages][2][block][H][D]
  const int32_t* page_ids;
  int H, D, block_size;
  int64_t kc_sb, kc_sn, kc_sh, vc_sb, vc_sn, vc_sh;
};

constexpr int kWireItems = 4;

template <bool TO_WIRE>
__global__ void __launch_bounds__(kThreads) wire_pages_kernel(const WireArgs a) {
  const int64_t p = blockIdx.x;
  const int per_row = a.D / 16, per_slot = a.H * per_row, per_side = a.block_size * per_slot;   // 16-byte items
  const int64_t page = __ldg(a.page_ids + p);
  int8_t* w = a.wire + p * 2 * per_side * 16;
  for (int base = threadIdx.x; base < 2 * per_side; base += kThreads * kWireItems) {
    uint4 v[kWireItems];
    int8_t* cp[kWireItems];
#pragma unroll
    for (int u = 0; u < kWireItems; ++u) {
      const int i = base + u * kThreads;
      cp[u] = nullptr;
      if (i < 2 * per_side) {
        const int side = i >= per_side, j = i - side * per_side;
        const int n = j / per_slot, rem = j - n * per_slot, h = rem / per_row, c = (rem - h * per_row) * 16;
        cp[u] = side ? a.vc + page * a.vc_sb + n * a.vc_sn + h * a.vc_sh + c : a.kc + page * a.kc_sb + n * a.kc_sn + h * a.kc_sh + c;
        v[u] = TO_WIRE ? ld_stream16(cp[u]) : ld_stream16(w + static_cast<int64_t>(i) * 16);
      }
    }
#pragma unroll
    for (int u = 0; u < kWireItems; ++u) {
      const int i = base + u * kThreads;
      if (cp[u]) *reinterpret_cast<uint4*>(TO_WIRE ? w + static_cast<int64_t>(i) * 16 : cp[u]) = v[u];
    }
  }
}

int wire_pages(bool to_wire, void* k_cache, void* v_cache, void* wire, const int32_t* page_ids, int64_t num_pages,
               int num_kv_heads, int head_dim, int block_size, int64_t kc_stride_b, int64_t kc_stride_n, int64_t kc_stride_h,
               int64_t vc_stride_b, int64_t vc_stride_n, int64_t vc_stride_h, kvq_stream_t stream) {
  KVQ_REQUIRE(head_dim > 0 && head_dim % 16 == 0, "wire pages: head_dim must be a multiple of 16, got %d", head_dim);
  KVQ_REQUIRE(num_kv_heads > 0 && block_size > 0, "wire pages: bad sizes");
  if (num_pages <= 0) return KVQ_OK;
  KVQ_REQUIRE(k_cache && v_cache && wire && page_ids, "wire pages: null pointer");
  KVQ_REQUIRE(aligned16(k_cache) && aligned16(v_cache) && aligned16(wire) && kc_stride_b % 16 == 0 && kc_stride_n % 16 == 0 &&
                  kc_stride_h % 16 == 0 && vc_stride_b % 16 == 0 && vc_stride_n % 16 == 0 && vc_stride_h % 16 == 0,
              "wire pages: rows must be 16-byte aligned");
  WireArgs a;
  a.kc = static_cast<int8_t*>(k_cache), a.vc = static_cast<int8_t*>(v_cache), a.wire = static_cast<int8_t*>(wire);
  a.page_ids = page_ids, a.H = num_kv_heads, a.D = head_dim, a.block_size = block_size;
  a.kc_sb = kc_stride_b, a.kc_sn = kc_stride_n, a.kc_sh = kc_stride_h;
  a.vc_sb = vc_stride_b, a.vc_sn = vc_stride_n, a.vc_sh = vc_stride_h;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (to_wire)
    wire_pages_kernel<true><<<static_cast<unsigned>(num_pages), kThreads, 0, s>>>(a);
  else
    wire_pages_kernel<false><<<static_cast<unsigned>(num_pages), kThreads, 0, s>>>(a);
  KVQ_CUDA(cudaGetLastError());
  return KVQ_OK;
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
  a.H = num_kv_heads, a.D = head_dim, a.groups = head_dim / 8;
  a.n_items = num_tokens * num_kv_heads * a.groups;
  a.block_size = block_size, a.bs_shift = ilog2_exact(block_size);
  a.k_st = key_stride_t, a.k_sh = key_stride_h, a.v_st = value_stride_t, a.v_sh = value_stride_h;
  a.kc_sb = kc_stride_b, a.kc_sn = kc_stride_n, a.kc_sh = kc_stride_h;
  a.vc_sb = vc_stride_b, a.vc_sn = vc_stride_n, a.vc_sh = vc_stride_h;
  a.pc_k = k_per_channel, a.pc_v = v_per_channel;
  const int64_t blocks = (a.n_items + kThreads * kItems - 1) / (kThreads * kItems);
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
  const int64_t blocks = (rows * 16 + kThreads - 1) / kThreads;
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
  a.H = num_kv_heads, a.D = head_dim, a.groups = head_dim / 8, a.block_size = block_size;
  a.bt_stride = bt_stride;
  a.kc_sb = kc_stride_b, a.kc_sn = kc_stride_n, a.kc_sh = kc_stride_h;
  a.vc_sb = vc_stride_b, a.vc_sn = vc_stride_n, a.vc_sh = vc_stride_h;
  a.pc_k = k_per_channel, a.pc_v = v_per_channel;
  dequant_pages_kernel<<<static_cast<unsigned>(num_pages), kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  KVQ_CUDA(cudaGetLastError());
  return KVQ_OK;
}

extern "C" __attribute__((visibility("default"))) int kvq_pages_to_wire(const void* k_cache, const void* v_cache, void* wire, const int32_t* page_ids,
                                 int64_t num_pages, int num_kv_heads, int head_dim, int block_size, int64_t kc_stride_b,
                                 int64_t kc_stride_n, int64_t kc_stride_h, int64_t vc_stride_b, int64_t vc_stride_n,
                                 int64_t vc_stride_h, kvq_stream_t stream) {
  return wire_pages(true, const_cast<void*>(k_cache), const_cast<void*>(v_cache), wire, page_ids, num_pages, num_kv_heads,
                    head_dim, block_size, kc_stride_b, kc_stride_n, kc_stride_h, vc_stride_b, vc_stride_n, vc_stride_h, stream);
}

extern "C" __attribute__((visibility("default"))) int kvq_wire_to_pages(const void* wire, void* k_cache, void* v_cache, const int32_t* page_ids,
                                 int64_t num_pages, int num_kv_heads, int head_dim, int block_size, int64_t kc_stride_b,
                                 int64_t kc_stride_n, int64_t kc_stride_h, int64_t vc_stride_b, int64_t vc_stride_n,
                                 int64_t vc_stride_h, kvq_stream_t stream) {
  return wire_pages(false, k_cache, v_cache, const_cast<void*>(wire), page_ids, num_pages, num_kv_heads, head_dim, block_size,
                    kc_stride_b, kc_stride_n, kc_stride_h, vc_stride_b, vc_stride_n, vc_stride_h, stream);
}
