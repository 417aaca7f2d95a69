// Long-query (prefill / chunked-prefill) causal attention that reads the INT8 paged cache directly, on sm_100a.
//
// The reference serves requests with more than SHORT_Q query tokens by dequantizing their pages into a temporary
// bf16 paged cache and running FlashAttention over it (kvq/cuda_kernels.py:61-131, "implementation A" of
// kvq/int8_ref.py:62-91). This kernel computes the same attention - bf16 q against K = k_i8 * s_k and
// V = v_i8 * s_v - from the int8 pages, without the temporary cache (and without its bf16 rounding of K and V):
//
//   prefill_plan_kernel   work items (pairs of m tiles) per long request, exclusive prefix (one block)
//   prefill_ws_kernel     one CTA per (request, kv head, pair of m tiles of 128 (token, q head) rows)
//
// q rows are loaded once, multiplied by s_k[channel] (exact fold: q.(k_i8 * s_k) = (q * s_k).k_i8), scaled by a
// per-row power of two into fp16 range and kept in shared memory as the A operand. K/V arrive as int8 16-key boxes
// by TMA (cp.async.bulk.tensor, mbarrier completion), are widened to fp16 (exact: |k_i8| <= 127) into
// 128-byte-swizzled operand tiles, and both products run on the 5th-generation tensor cores:
//   S[128 x 128]  = Q . K^T    tcgen05.mma kind::f16, A and B K-major from shared memory, fp32 accumulator in TMEM
//   O[128 x D]   += P . V      P fp16 from tensor memory, V MN-major (its natural [key][channel] layout) from smem
// Each softmax thread reads its own row of S from TMEM (tcgen05.ld), does the online softmax in fp32 with the
// running maximum held back until it grows by more than 2^8 (the accumulator in TMEM is rescaled only then), and
// writes its P row back to TMEM. s_v and 1 / denominator are applied once in the epilogue. All waits are bounded;
// a wait that expires sets the status word in the workspace and the CTA leaves after releasing its tensor memory.
#include <cuda.h>
#include <cuda_fp16.h>

#include "kvq_common.cuh"
#include "kvq_host.h"
#include "kvq_ptx.cuh"

namespace kvq {
namespace {

constexpr int PF_BM = 128;         // rows per m tile: (query token, q head of the kv head's group), one thread each
constexpr int PF_HDR_BYTES = 256;  // workspace header: int32 [0] status, [1] work items (pairs of m tiles)

struct PrefillArgs {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  const int32_t *cu_q, *seq_lens, *block_table;
  const float *ks, *vs;
  int32_t* hdr;
  int32_t* prefix;       // [num_seqs + 1] exclusive prefix of m tiles per request
  float scale_log2;      // softmax scale * log2(e)
  int num_seqs, Hkv, G, TQ, lbs, bs_mask, min_q;   // TQ: query tokens per m tile; requests with q_len <= min_q are skipped
  int64_t q_st, q_sh, o_st, o_sh, bt_stride;
  int pc_k, pc_v;
  int kpos[3], vpos[3];  // tensor-map coordinate slot (1..3) of the (slot-in-block, head, block) dims
};

// ------------------------------------------------------------------------------------------------------
// tcgen05 (kind::f16) pieces specific to this kernel
// ------------------------------------------------------------------------------------------------------
// D[tmem] (+)= A[smem] . B[smem]; issued by one thread.
__device__ __forceinline__ void umma_f16(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Instruction descriptor of kind::f16: fp16 A and B, fp32 accumulator, M x N tile, B MN-major or K-major.
__host__ __device__ constexpr uint32_t instr_desc(int M, int N, bool b_mn_major) {
  return (1u << 4) | (b_mn_major ? (1u << 16) : 0u) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}
// Byte offset of the 16-byte chunk `c16` of row `r` inside a swizzled [rows][128 B] slab.
__device__ __forceinline__ uint32_t slab_off(int r, int c16) { return r * 128 + ((c16 ^ (r & 7)) << 4); }

// Four int8 -> four fp16, exact: byte ^ 0x80 is the value + 128 as an unsigned byte; 0x6400 | byte is the fp16
// 1024 + byte; subtracting 1152 leaves the value.
__device__ __forceinline__ void i8x4_to_f16x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t u = w ^ 0x80808080u;
  const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
  uint32_t a = __byte_perm(u, 0x64646464u, 0x4140), b = __byte_perm(u, 0x64646464u, 0x4342);
  const __half2 x = __hsub2(*reinterpret_cast<const __half2*>(&a), bias);
  const __half2 y = __hsub2(*reinterpret_cast<const __half2*>(&b), bias);
  lo = *reinterpret_cast<const uint32_t*>(&x);
  hi = *reinterpret_cast<const uint32_t*>(&y);
}
// Packed fp32 pairs (sm_100: fma.rn.f32x2 is two IEEE operations in one instruction).
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 pk2(float a, float b) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void upk2(f32x2 v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// ------------------------------------------------------------------------------------------------------
// plan: m tiles per request (long requests only), exclusive prefix
// ------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) prefill_plan_kernel(const int32_t* __restrict__ cu_q, int num_seqs, int TQ, int min_q,
                                                          int per_cta, int32_t* __restrict__ hdr,
                                                          int32_t* __restrict__ prefix) {
  __shared__ int s_warp[8];
  __shared__ int s_carry;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_carry = 0, hdr[0] = 0;
  __syncthreads();
  for (int base = 0; base < num_seqs; base += 256) {
    const int r = base + tid;
    int n = 0;
    if (r < num_seqs) {
      const int qlen = cu_q[r + 1] - cu_q[r];
      n = qlen > min_q ? ((qlen + TQ - 1) / TQ + per_cta - 1) / per_cta : 0;
    }
    int incl = n;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += y;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    int before = s_carry;
    for (int w = 0; w < warp; ++w) before += s_warp[w];
    if (r < num_seqs) prefix[r] = before + incl - n;
    __syncthreads();
    if (tid == 255) s_carry = before + incl;
    __syncthreads();
  }
  if (tid == 0) prefix[num_seqs] = s_carry, hdr[1] = s_carry;
}

// ------------------------------------------------------------------------------------------------------
// warp-specialized kernel: two m tiles per CTA share one K/V stream
// ------------------------------------------------------------------------------------------------------
// 14 warps: warps 0-3 and 4-7 are the softmax groups of m tile 0 and 1 (one thread per row), warps 8-11 widen the
// int8 K/V boxes into fp16 operand tiles, warp 12 (one lane) issues every tcgen05.mma, warp 13 the TMA loads.
// The groups meet only through mbarriers. Steps are 128 keys. Per m tile the chain is S = Q.K^T -> softmax ->
// O += P.V; the tensor core works on one tile's products while the other tile is in its softmax (the two chains run
// half a step apart), and the converters run up to two steps ahead.
//   TMEM (512 columns): S[tile] 2 x 128 fp32 columns, O[tile] 2 x D. P (fp16 pairs, 64 columns) is written over the
//     first half of its tile's S and is the A operand of P.V straight from tensor memory.
//   smem: Q 2 tiles, fp16 K and V 2 stages each, one int8 landing zone each for K and V.
// A tcgen05.mma of 128 x N x 16 with N <= 128 occupies the tensor core for ~90 cycles however small N is (measured),
// so steps of 128 keys (N = 128 for S) halve the cost of S against 64-key steps.
constexpr int WS_BN = 128;           // keys per step
constexpr int WS_THREADS = 14 * 32;
constexpr int WS_TMEM_COLS = 512;
enum WsBar {
  WB_STGK = 0,        // int8 K boxes of a step landed (TMA)
  WB_STGV = 1,
  WB_STGK_FREE = 2,   // landing zone read by every converter (128 threads)
  WB_STGV_FREE = 3,
  WB_KF_READY = 4,    // [2] fp16 K tile written (128 converter threads)
  WB_VF_READY = 6,    // [2]
  WB_KF_FREE = 8,     // [2] tensor core done with the fp16 K tile (commit)
  WB_VF_FREE = 10,    // [2]
  WB_S_READY = 12,    // [tile] S of the step computed (commit)
  WB_P_READY = 14,    // [tile * 2 + half] P of 64 keys of the step written to tensor memory (128 softmax threads)
  WB_O_DONE = 18,     // [tile] O += P.V of the step finished (commit)
  WB_Q_READY = 20,    // q tiles written (256 softmax threads)
  WB_COUNT = 21
};

template <int D>
struct WsGeom {
  static constexpr int NSLAB = D / 64;
  static constexpr int Q_TILE = NSLAB * PF_BM * 128;
  static constexpr int KV_SLAB = WS_BN * 128;      // [128 keys][64 channels] fp16
  static constexpr int KV_TILE = NSLAB * KV_SLAB;
  static constexpr int STG = WS_BN * D;            // int8 landing zone of one K or V step (eight 16-key boxes)
  static constexpr int OFF_Q = 0, OFF_K = OFF_Q + 2 * Q_TILE, OFF_V = OFF_K + 2 * KV_TILE, OFF_SK = OFF_V + 2 * KV_TILE,
                       OFF_SV = OFF_SK + STG, END = OFF_SV + STG;
  static constexpr int SMEM = 1024 + END;
};

// int8 landing zone (TMA boxes of [16 keys][D bytes], hardware-swizzled) of WS_BN keys -> fp16 operand slabs.
// 16 channels per item; called by the 128 converter threads.
template <int D>
__device__ __forceinline__ void widen_step(const uint8_t* __restrict__ stg, uint8_t* __restrict__ dst, int tid) {
  constexpr int CPR = D / 16, N = WS_BN * CPR / 128;
  uint4 w[N];
#pragma unroll
  for (int i = 0; i < N; ++i) {   // every load before the first conversion
    const int idx = tid + 128 * i, key = idx / CPR, c = idx - key * CPR, kk = key & 15;
    w[i] = *reinterpret_cast<const uint4*>(stg + (key >> 4) * 16 * D + kk * D +
                                           ((D == 128 ? (c ^ (kk & 7)) : (c ^ ((kk >> 1) & 3))) << 4));
  }
#pragma unroll
  for (int i = 0; i < N; ++i) {
    const int idx = tid + 128 * i, key = idx / CPR, c = idx - key * CPR;
    uint4 lo, hi;
    i8x4_to_f16x4(w[i].x, lo.x, lo.y);
    i8x4_to_f16x4(w[i].y, lo.z, lo.w);
    i8x4_to_f16x4(w[i].z, hi.x, hi.y);
    i8x4_to_f16x4(w[i].w, hi.z, hi.w);
    uint8_t* slab = dst + (c >> 2) * WsGeom<D>::KV_SLAB;
    *reinterpret_cast<uint4*>(slab + slab_off(key, (c & 3) * 2)) = lo;
    *reinterpret_cast<uint4*>(slab + slab_off(key, (c & 3) * 2 + 1)) = hi;
  }
}

// D[tmem] (+)= A[tmem] . B[smem]: A is 128 lanes x 8 columns of packed fp16 pairs (k = 2 * column, 2 * column + 1).
__device__ __forceinline__ void umma_f16_ts(uint32_t d, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(addr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

template <int D>
__global__ void __launch_bounds__(WS_THREADS, 1)
    prefill_ws_kernel(const PrefillArgs a, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
  using Gm = WsGeom<D>;
  constexpr int NSLAB = Gm::NSLAB;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_bar[WB_COUNT];
  __shared__ uint32_t s_tmem;
  __shared__ int s_req;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_wait();   // the plan below is written by prefill_plan_kernel
  const int total = a.hdr[1];   // pairs of m tiles
  const int pix = blockIdx.x / a.Hkv, kvh = blockIdx.x - pix * a.Hkv;
  if (pix >= total) return;
  const int pair = total - 1 - pix;   // later m tiles of a request see more keys: start them first

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* p_base = smem_raw + (base - smem_u32(smem_raw));
  auto bar = [&](int i) { return smem_u32(&s_bar[i]); };

  if (warp == 12) tmem_alloc(smem_u32(&s_tmem), WS_TMEM_COLS);
  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < WB_COUNT; ++i) {
      const bool by_group = i == WB_STGK_FREE || i == WB_STGV_FREE || (i >= WB_KF_READY && i < WB_KF_FREE) ||
                            (i >= WB_P_READY && i < WB_O_DONE);   // arrivals from a 128-thread group
      mbar_init(bar(i), by_group ? 128 : (i == WB_Q_READY ? 256 : 1));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int r = tid; r < a.num_seqs; r += WS_THREADS)
    if (a.prefix[r] <= pair && pair < a.prefix[r + 1]) s_req = r;
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  volatile int* abort_flag = &s_abort;

  const int req = s_req, mt0 = 2 * (pair - a.prefix[req]);
  const int tok0 = a.cu_q[req], qlen = a.cu_q[req + 1] - tok0, L = a.seq_lens[req];
  const int32_t* bt = a.block_table + static_cast<int64_t>(req) * a.bt_stride;
  // key steps of each m tile: tile t covers query tokens [t_first, t_last]; keys [0, L - qlen + 1 + t_last) are visible
  auto steps_of = [&](int mt) {
    const int t_first = mt * a.TQ;
    if (t_first >= qlen) return 0;
    const int kmax = L - qlen + 1 + min(qlen, t_first + a.TQ) - 1;
    return kmax > 0 ? (kmax + WS_BN - 1) / WS_BN : 0;
  };
  const int nk0 = steps_of(mt0), nk1 = steps_of(mt0 + 1), nk = max(nk0, nk1);
  constexpr uint32_t ID_S = instr_desc(PF_BM, WS_BN, false), ID_O = instr_desc(PF_BM, D, true);

  if (warp < 8) {
    // ================= softmax group of m tile t =================
    const int t = warp >> 2, row = tid & 127, mt = mt0 + t, nkt = t ? nk1 : nk0;
    uint8_t* p_q = p_base + Gm::OFF_Q + t * Gm::Q_TILE;
    const uint32_t t_lane = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem + t * WS_BN + t_lane, t_o = tmem + 2 * WS_BN + t * D + t_lane;
    const int tl = row / a.G, hg = row - tl * a.G, tq = mt * a.TQ + tl;
    const bool valid = tl < a.TQ && tq < qlen;
    const int lim = valid ? L - qlen + 1 + tq : 0x7fffffff;   // padding rows hold q = 0 and are never stored
    float c_row = 0.f;
    {
      const __nv_bfloat16* qrow = a.q + static_cast<int64_t>(tok0 + tq) * a.q_st + static_cast<int64_t>(kvh * a.G + hg) * a.q_sh;
      const float* ksr = a.ks + kvh * (a.pc_k ? D : 1);
      // 8 loads (128 bytes of the row) are in flight per round trip; the second pass finds the row in L1 / L2
      auto scaled = [&](const uint4& w, int c, float (&f)[8]) {   // channels 8c..8c+7 of q * s_k
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) f[2 * e] = bf16lo(ww[e]), f[2 * e + 1] = bf16hi(ww[e]);
        if (a.pc_k) {
          const float4 s0 = __ldg(reinterpret_cast<const float4*>(ksr) + 2 * c), s1 = __ldg(reinterpret_cast<const float4*>(ksr) + 2 * c + 1);
          f[0] *= s0.x, f[1] *= s0.y, f[2] *= s0.z, f[3] *= s0.w, f[4] *= s1.x, f[5] *= s1.y, f[6] *= s1.z, f[7] *= s1.w;
        }
      };
      float amax = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < D / 8; c0 += 8) {
        uint4 raw[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) raw[i] = valid ? __ldg(reinterpret_cast<const uint4*>(qrow) + c0 + i) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float f[8];
          scaled(raw[i], c0 + i, f);
#pragma unroll
          for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
        }
      }
      // power-of-two row scale that puts the largest |q * s_k| into [2^14, 2^15): fp16 keeps 11 significant bits
      int ex = 0;
      if (amax > 0.f) frexpf(amax, &ex);
      const int sh = amax > 0.f ? max(-60, min(60, 15 - ex)) : 0;
      const float up = ldexpf(1.f, sh);
      c_row = a.scale_log2 * ldexpf(1.f, -sh) * (a.pc_k ? 1.f : __ldg(ksr));
#pragma unroll 1
      for (int c0 = 0; c0 < D / 8; c0 += 8) {
        uint4 raw[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) raw[i] = valid ? __ldg(reinterpret_cast<const uint4*>(qrow) + c0 + i) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float f[8];
          scaled(raw[i], c0 + i, f);   // zeros for a padding row
          const int c = c0 + i;
          *reinterpret_cast<uint4*>(p_q + (c >> 3) * (PF_BM * 128) + slab_off(row, c & 7)) =
              make_uint4(pack_f16x2(f[0] * up, f[1] * up), pack_f16x2(f[2] * up, f[3] * up), pack_f16x2(f[4] * up, f[5] * up),
                         pack_f16x2(f[6] * up, f[7] * up));
        }
      }
    }
    fence_proxy_async();
    mbar_arrive(bar(WB_Q_READY));

    float m_ref = -1e30f, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < nkt && ok; ++j) {
      ok = ws_wait(bar(WB_S_READY + t), j & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      // pass 1: row maximum of the step's 128 scores (64 columns per round trip to tensor memory)
      const int n_base = j * WS_BN;
      const bool masked = n_base + WS_BN > lim;
      float mx = -INFINITY;
      {
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < WS_BN; c += 64) {
          uint32_t sa[32], sb[32];
          tmem_ld32(t_s + c, sa);
          tmem_ld32(t_s + c + 32, sb);
          tmem_wait_ld();
          if (!masked) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              m4[(i >> 1) & 3] = fmaxf(m4[(i >> 1) & 3], fmaxf(__uint_as_float(sa[i]), __uint_as_float(sa[i + 1])));
              m4[(i >> 1) & 3] = fmaxf(m4[(i >> 1) & 3], fmaxf(__uint_as_float(sb[i]), __uint_as_float(sb[i + 1])));
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (n_base + c + i < lim) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(sa[i]));
              if (n_base + c + 32 + i < lim) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(sb[i]));
            }
          }
        }
        mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      }
      const float tile_max = mx * c_row;   // c_row > 0
      const bool grow = tile_max > m_ref + 8.f;
      float alpha = 1.f;
      if (grow) {
        alpha = ex2(m_ref - tile_max);   // 0 on the first step (m_ref = -1e30)
        m_ref = tile_max;
        l_sum *= alpha;
      }
      // S of this step is committed after O += P.V of the previous step, so O may be rescaled here
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t o[32];
          tmem_ld32(t_o + c, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(t_o + c, o);
        }
      }
      // pass 2: P = exp2(S * c_row - m_ref) as fp16 pairs, written over the first half of S chunk by chunk
      // (chunk i reads S columns [32 i, 32 i + 32) and then writes P columns [16 i, 16 i + 16): never ahead of a
      // read). P.V may start on the first 64 keys while the last 64 are still being computed.
      {
        const f32x2 c2 = pk2(c_row, c_row), nm2 = pk2(-m_ref, -m_ref);
        float ls = 0.f;
#pragma unroll 1
        for (int c = 0; c < WS_BN; c += 32) {
          uint32_t sr[32];
          tmem_ld32(t_s + c, sr);
          tmem_wait_ld();
          uint32_t w[16];
          f32x2 ls2 = pk2(0.f, 0.f);
          if (!masked) {   // every step but the last ones of a row
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float x0, x1;
              upk2(fma2(pk2(__uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1])), c2, nm2), x0, x1);
              const float p0 = ex2(x0), p1 = ex2(x1);
              ls2 = add2(ls2, pk2(p0, p1));
              w[i] = pack_f16x2(p0, p1);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float x0, x1;
              upk2(fma2(pk2(__uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1])), c2, nm2), x0, x1);
              const float p0 = n_base + c + 2 * i < lim ? ex2(x0) : 0.f;
              const float p1 = n_base + c + 2 * i + 1 < lim ? ex2(x1) : 0.f;
              ls2 = add2(ls2, pk2(p0, p1));
              w[i] = pack_f16x2(p0, p1);
            }
          }
          {
            float a0, a1;
            upk2(ls2, a0, a1);
            ls += a0 + a1;
          }
          tmem_st16(t_s + (c >> 1), w);
          if (c & 32) {   // 64 keys of P complete
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar(WB_P_READY + t * 2 + (c >> 6)));
          }
        }
        l_sum += ls;
      }
    }
    // ---- epilogue: O / denominator * s_v -> bf16 ----
    if (ok && nkt > 0) ok = ws_wait(bar(WB_O_DONE + t), (nkt - 1) & 1, abort_flag);
    if (ok && nkt > 0) {
      tc_fence_after();
      __nv_bfloat16* orow = a.out + static_cast<int64_t>(tok0 + tq) * a.o_st + static_cast<int64_t>(kvh * a.G + hg) * a.o_sh;
      const float inv = 1.f / fmaxf(l_sum, 1e-30f);
      const float* vsr = a.vs + kvh * (a.pc_v ? D : 1);
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t o[32];
        tmem_ld32(t_o + c, o);
        tmem_wait_ld();
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            float sv[8];
            if (a.pc_v) {
              const float4 s0 = __ldg(reinterpret_cast<const float4*>(vsr + c + i)), s1 = __ldg(reinterpret_cast<const float4*>(vsr + c + i + 4));
              sv[0] = s0.x, sv[1] = s0.y, sv[2] = s0.z, sv[3] = s0.w, sv[4] = s1.x, sv[5] = s1.y, sv[6] = s1.z, sv[7] = s1.w;
            } else {
              const float one = __ldg(vsr);
#pragma unroll
              for (int e = 0; e < 8; ++e) sv[e] = one;
            }
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
              w[e] = pack_bf16x2(__uint_as_float(o[i + 2 * e]) * inv * sv[2 * e], __uint_as_float(o[i + 2 * e + 1]) * inv * sv[2 * e + 1]);
            *reinterpret_cast<uint4*>(orow + c + i) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    } else if (valid && nkt == 0) {   // no visible key (seq_len < q_len): defined output
      __nv_bfloat16* orow = a.out + static_cast<int64_t>(tok0 + tq) * a.o_st + static_cast<int64_t>(kvh * a.G + hg) * a.o_sh;
      for (int c = 0; c < D; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0u, 0u, 0u, 0u);
    }
  } else if (warp < 12) {
    // ================= converters: int8 -> fp16 =================
    const int ctid = tid - 256;
    bool ok = true;
    for (int j = 0; j < nk && ok; ++j) {
      const int s = j & 1;
      ok = ws_wait(bar(WB_STGK), j & 1, abort_flag);
      if (ok && j >= 2) ok = ws_wait(bar(WB_KF_FREE + s), ((j - 2) >> 1) & 1, abort_flag);
      if (!ok) break;
      widen_step<D>(p_base + Gm::OFF_SK, p_base + Gm::OFF_K + s * Gm::KV_TILE, ctid);
      fence_proxy_async();
      mbar_arrive(bar(WB_KF_READY + s));
      mbar_arrive(bar(WB_STGK_FREE));   // the landing zone may be refilled (producer warp)
      ok = ws_wait(bar(WB_STGV), j & 1, abort_flag);
      if (ok && j >= 2) ok = ws_wait(bar(WB_VF_FREE + s), ((j - 2) >> 1) & 1, abort_flag);
      if (!ok) break;
      widen_step<D>(p_base + Gm::OFF_SV, p_base + Gm::OFF_V + s * Gm::KV_TILE, ctid);
      fence_proxy_async();
      mbar_arrive(bar(WB_VF_READY + s));
      mbar_arrive(bar(WB_STGV_FREE));
    }
  } else if (warp == 13) {
    // ================= TMA producer: lane i < 8 loads the i-th 16-key box of a step =================
    auto key_of = [&](int j) {   // first key of this lane's box of step j; boxes past the end re-read the first
      const int n0 = j * WS_BN, n = n0 + 16 * lane;
      return n < L ? n : n0;
    };
    auto issue = [&](bool is_k, int j, int page) {
      const uint32_t full = bar(is_k ? WB_STGK : WB_STGV);
      if (lane == 0) mbar_expect_tx(full, Gm::STG);
      __syncwarp();
      if (lane < 8) {
        const int off = key_of(j) & a.bs_mask;
        const int* pos = is_k ? a.kpos : a.vpos;
        auto coord = [&](int s) { return pos[0] == s ? off : (pos[1] == s ? kvh : page); };
        tma_load_4d(base + (is_k ? Gm::OFF_SK : Gm::OFF_SV) + lane * 16 * D, is_k ? &tm_k : &tm_v, 0, coord(1), coord(2),
                    coord(3), full);
      }
    };
    int pg_a = 0, pg_b = 0;   // page ids (lanes 0-7) of the next two steps to issue
    if (lane < 8 && nk > 0) pg_a = bt[key_of(0) >> a.lbs];
    if (nk > 0) issue(true, 0, pg_a), issue(false, 0, pg_a);
    pg_a = pg_b = 0;
    if (lane < 8) {
      if (nk > 1) pg_a = bt[key_of(1) >> a.lbs];
      if (nk > 2) pg_b = bt[key_of(2) >> a.lbs];
    }
    bool ok = true;
    for (int j = 0; j + 1 < nk && ok; ++j) {
      // pg_a belongs to step j + 1, pg_b to step j + 2; a landing zone is refilled once every converter has read it
      ok = ws_wait(bar(WB_STGK_FREE), j & 1, abort_flag);
      if (ok) issue(true, j + 1, pg_a);
      ok = ok && ws_wait(bar(WB_STGV_FREE), j & 1, abort_flag);
      if (ok) issue(false, j + 1, pg_a);
      pg_a = pg_b;
      pg_b = (lane < 8 && j + 3 < nk) ? bt[key_of(j + 3) >> a.lbs] : 0;
    }
  } else if (warp == 12 && lane == 0) {
    // ================= tensor-core issue (one thread) =================
    bool ok = ws_wait_thread(bar(WB_Q_READY), 0, abort_flag);
    // Descriptors differ only in their 14-bit start-address field (address >> 4): one base per operand, the
    // tile / slab / k-step offsets (compile-time constants once the loops are unrolled) are added to it.
    const uint64_t d_q = smem_desc(base + Gm::OFF_Q, 16, 1024), d_k = smem_desc(base + Gm::OFF_K, 16, 1024),
                   d_v = smem_desc(base + Gm::OFF_V, Gm::KV_SLAB, 1024);
    auto issue_qk = [&](int t, int j) {   // S[t] = Q[t] . K(j)^T
      const int s = j & 1;
      ok = ok && ws_wait_thread(bar(WB_KF_READY + s), (j >> 1) & 1, abort_flag);
      if (!ok) return;
      tc_fence_after();
      const uint64_t d_ks = d_k + static_cast<uint64_t>((s * Gm::KV_TILE) >> 4);
      const uint64_t d_qt = d_q + static_cast<uint64_t>((t * Gm::Q_TILE) >> 4);
#pragma unroll
      for (int sl = 0; sl < NSLAB; ++sl)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_f16(tmem + t * WS_BN, d_qt + static_cast<uint64_t>((sl * (PF_BM * 128) + ks * 32) >> 4),
                   d_ks + static_cast<uint64_t>((sl * Gm::KV_SLAB + ks * 32) >> 4), ID_S, (sl | ks) ? 1u : 0u);
      umma_commit(bar(WB_S_READY + t));
    };
    if (ok && nk0 > 0) issue_qk(0, 0);
    if (ok && nk1 > 0) issue_qk(1, 0);
    if (ok && nk > 0) umma_commit(bar(WB_KF_FREE));
    for (int j = 0; j < nk && ok; ++j) {
      const int s = j & 1;
      ok = ws_wait_thread(bar(WB_VF_READY + s), (j >> 1) & 1, abort_flag);
      const uint64_t d_vs = d_v + static_cast<uint64_t>((s * Gm::KV_TILE) >> 4);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int nkt = t ? nk1 : nk0;
        if (!ok || j >= nkt) continue;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          ok = ok && ws_wait_thread(bar(WB_P_READY + t * 2 + h), j & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int ks = 4 * h; ks < 4 * h + 4; ++ks)   // 16 keys = 8 columns of packed P per k step
            umma_f16_ts(tmem + 2 * WS_BN + t * D, tmem + t * WS_BN + ks * 8,
                        d_vs + static_cast<uint64_t>((ks * 16 * 128) >> 4), ID_O, (j | ks) ? 1u : 0u);
        }
        if (!ok) continue;
        umma_commit(bar(WB_O_DONE + t));
        if (j + 1 < nkt) issue_qk(t, j + 1);   // executes after the P.V above: S[t] (and the P inside it) is free again
      }
      if (ok) {
        umma_commit(bar(WB_VF_FREE + s));
        if (j + 1 < nk) umma_commit(bar(WB_KF_FREE + (s ^ 1)));
      }
    }
  }

  // ---- common exit ----
  if (*abort_flag) {
    // A bounded wait expired somewhere in the CTA: report it and give copies and tensor-core work still in flight
    // a bounded time to land before shared and tensor memory are released.
    if (tid == 0) atomicExch(a.hdr, 1);
    const long long t0 = clock64();
    while (clock64() - t0 < (1ll << 20)) __nanosleep(256);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 12) tmem_dealloc(tmem, WS_TMEM_COLS);
}

// ------------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------------
size_t pf_align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

template <typename... KArgs, typename... Args>
cudaError_t pf_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

bool g_pf_ready[64] = {};

}  // namespace
}  // namespace kvq

using namespace kvq;

extern "C" __attribute__((visibility("default"))) size_t kvq_prefill_workspace_size(int num_seqs) {
  if (num_seqs < 0) return 0;
  return PF_HDR_BYTES + pf_align_up(static_cast<size_t>(num_seqs + 1) * 4, 256);
}

extern "C" __attribute__((visibility("default"))) int kvq_int8_prefill_attention(
    const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* cu_q, const int32_t* seq_lens,
    const int32_t* block_table, const float* k_scale, const float* v_scale, double softmax_scale, int num_seqs,
    int64_t total_query_tokens, int num_q_heads, int num_kv_heads, int head_dim, int block_size, int64_t num_blocks,
    int64_t q_stride_t, int64_t q_stride_h, int64_t o_stride_t, int64_t o_stride_h, int64_t kc_stride_b, int64_t kc_stride_n,
    int64_t kc_stride_h, int64_t vc_stride_b, int64_t vc_stride_n, int64_t vc_stride_h, int64_t bt_stride, int k_per_channel,
    int v_per_channel, int min_query_len, void* workspace, size_t workspace_bytes, kvq_stream_t stream) {
  if (num_seqs == 0 || total_query_tokens == 0) return KVQ_OK;
  KVQ_REQUIRE(q && k_cache && v_cache && out && cu_q && seq_lens && block_table && k_scale && v_scale && workspace,
              "prefill_attention: null pointer");
  KVQ_REQUIRE(num_seqs > 0 && total_query_tokens > 0 && min_query_len >= 0, "prefill_attention: bad sizes");
  KVQ_REQUIRE(head_dim == 64 || head_dim == 128, "prefill_attention: head_dim must be 64 or 128, got %d", head_dim);
  KVQ_REQUIRE(num_kv_heads > 0 && num_q_heads % num_kv_heads == 0 && num_q_heads / num_kv_heads <= PF_BM,
              "prefill_attention: %d q heads do not group over %d kv heads", num_q_heads, num_kv_heads);
  KVQ_REQUIRE(block_size >= 16 && (block_size & (block_size - 1)) == 0,
              "prefill_attention: block_size must be a power of two >= 16, got %d", block_size);
  KVQ_REQUIRE(aligned16(q) && aligned16(out) && q_stride_t % 8 == 0 && q_stride_h % 8 == 0 && o_stride_t % 8 == 0 &&
                  o_stride_h % 8 == 0,
              "prefill_attention: q / out rows must be 16-byte aligned");
  KVQ_REQUIRE(aligned16(k_cache) && aligned16(v_cache) && kc_stride_b % 16 == 0 && kc_stride_n % 16 == 0 &&
                  kc_stride_h % 16 == 0 && vc_stride_b % 16 == 0 && vc_stride_n % 16 == 0 && vc_stride_h % 16 == 0,
              "prefill_attention: cache base and strides must be multiples of 16 bytes");
  KVQ_REQUIRE(aligned16(k_scale) && aligned16(v_scale), "prefill_attention: scales must be 16-byte aligned");
  KVQ_REQUIRE(softmax_scale > 0.0, "prefill_attention: softmax_scale must be positive");
  if (workspace_bytes < kvq_prefill_workspace_size(num_seqs)) {
    set_error("prefill_attention: workspace of %zu bytes, %zu needed", workspace_bytes, kvq_prefill_workspace_size(num_seqs));
    return KVQ_ERR_WORKSPACE;
  }
  auto s = reinterpret_cast<cudaStream_t>(stream);
  int sms = 0, rc;
  if ((rc = shared_device_sms(&sms)) != KVQ_OK) return rc;
  int dev = 0;
  KVQ_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !g_pf_ready[dev]) {
    KVQ_CUDA(cudaFuncSetAttribute(prefill_ws_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, WsGeom<64>::SMEM));
    KVQ_CUDA(cudaFuncSetAttribute(prefill_ws_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, WsGeom<128>::SMEM));
    g_pf_ready[dev] = true;
  }

  PrefillArgs a = {};
  a.q = static_cast<const __nv_bfloat16*>(q), a.out = static_cast<__nv_bfloat16*>(out);
  a.cu_q = cu_q, a.seq_lens = seq_lens, a.block_table = block_table, a.ks = k_scale, a.vs = v_scale;
  a.hdr = static_cast<int32_t*>(workspace);
  a.prefix = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) + PF_HDR_BYTES);
  a.scale_log2 = static_cast<float>(softmax_scale * 1.4426950408889634);
  a.num_seqs = num_seqs, a.Hkv = num_kv_heads, a.G = num_q_heads / num_kv_heads, a.TQ = PF_BM / a.G;
  a.lbs = 0;
  while ((1 << a.lbs) < block_size) ++a.lbs;
  a.bs_mask = block_size - 1, a.min_q = min_query_len;
  a.q_st = q_stride_t, a.q_sh = q_stride_h, a.o_st = o_stride_t, a.o_sh = o_stride_h, a.bt_stride = bt_stride;
  a.pc_k = k_per_channel ? 1 : 0, a.pc_v = v_per_channel ? 1 : 0;
  CUtensorMap tm_k, tm_v;
  if ((rc = shared_cache_tensor_map(k_cache, num_blocks, block_size, num_kv_heads, head_dim, kc_stride_b, kc_stride_n,
                                    kc_stride_h, 1, &tm_k, a.kpos)) != KVQ_OK)
    return rc;
  if ((rc = shared_cache_tensor_map(v_cache, num_blocks, block_size, num_kv_heads, head_dim, vc_stride_b, vc_stride_n,
                                    vc_stride_h, 1, &tm_v, a.vpos)) != KVQ_OK)
    return rc;

  constexpr int per_cta = 2;   // m tiles per CTA
  prefill_plan_kernel<<<1, 256, 0, s>>>(cu_q, num_seqs, a.TQ, a.min_q, per_cta, a.hdr, a.prefix);
  KVQ_CUDA(cudaGetLastError());
  // upper bound of the work items: sum over requests of ceil(m tiles / per_cta), m tiles = ceil(q_len / TQ)
  const int64_t max_items = total_query_tokens / (static_cast<int64_t>(a.TQ) * per_cta) + num_seqs;
  KVQ_REQUIRE(max_items * num_kv_heads < (1ll << 31), "prefill_attention: batch too large");
  const dim3 grid(static_cast<unsigned>(max_items * num_kv_heads));
  if (head_dim == 128)
    KVQ_CUDA(pf_launch_pdl(prefill_ws_kernel<128>, grid, dim3(WS_THREADS), WsGeom<128>::SMEM, s, a, tm_k, tm_v));
  else
    KVQ_CUDA(pf_launch_pdl(prefill_ws_kernel<64>, grid, dim3(WS_THREADS), WsGeom<64>::SMEM, s, a, tm_k, tm_v));
  return KVQ_OK;
}

