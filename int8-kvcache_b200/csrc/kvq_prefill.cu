// Long-query (prefill / chunked-prefill) causal attention that reads the INT8 paged cache directly, on sm_100a.
//
// The reference serves requests with more than SHORT_Q query tokens by dequantizing their pages into a temporary
// bf16 paged cache and running FlashAttention over it (kvq/cuda_kernels.py:61-131, "implementation A" of
// kvq/int8_ref.py:62-91); its authors list the per-layer copy as the path's main cost (docs/WALKTHROUGH.md:408-409).
// This kernel computes the same attention - bf16 q against K = k_i8 * s_k and V = v_i8 * s_v - without the copy:
//
//   prefill_plan_kernel   m tiles per long request, exclusive prefix (one block)
//   prefill_kernel        one CTA per (request, kv head, m tile of 128 (token, q head) rows); 128 threads, one per row
//
// Per CTA: q rows are loaded once, multiplied by s_k[channel] (exact fold: q.(k_i8 * s_k) = (q * s_k).k_i8),
// scaled by a per-row power of two into fp16 range and kept in shared memory as the A operand. K/V arrive as int8
// 16-key boxes by TMA (cp.async.bulk.tensor, mbarrier completion), are widened to fp16 (exact: |k_i8| <= 127)
// into 128-byte-swizzled operand tiles, and both products run on the 5th-generation tensor cores:
//   S[128 x 64]   = Q . K^T    tcgen05.mma kind::f16, A and B K-major from shared memory, fp32 accumulator in TMEM
//   O[128 x D]   += P . V      P fp16 from shared memory (K-major), V MN-major (its natural [key][channel] layout)
// Each thread reads its own row of S from TMEM (tcgen05.ld), does the online softmax in fp32 with the running
// maximum held back until it grows by more than 2^8 (the accumulator in TMEM is rescaled only then), and writes
// its P row. s_v and 1 / denominator are applied once in the epilogue. All waits are bounded; a wait that expires
// sets the status word in the workspace and the CTA leaves after releasing its tensor memory.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "kvq_common.cuh"
#include "kvq_host.h"
#include "kvq_ptx.cuh"

namespace kvq {
namespace {

constexpr int PF_BM = 128;        // rows per CTA: (query token, q head of the kv head's group), one thread each
constexpr int PF_BN = 64;         // keys per step
constexpr int PF_THREADS = 128;
constexpr int PF_TMEM_COLS = 256;  // S: columns [0, 64), O: columns [64, 64 + D)
constexpr int PF_HDR_BYTES = 256;  // workspace header: int32 [0] status, [1] total m tiles

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
// tcgen05 wrappers
// ------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] (+)= A[smem] . B[smem]; issued by one thread.
__device__ __forceinline__ void umma_f16(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier receives one arrival when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 consecutive columns of this thread's TMEM lane (lane = 32 * (warp % 4) + lane id).
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
      "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(addr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
      "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(addr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
      "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
      "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle. Operand tiles are slabs of [rows][128 bytes] (64 fp16 per row)
// whose 16-byte chunks are XOR-swizzled with (row & 7); groups of 8 rows are 1024 bytes apart (stride byte offset).
// K-major operands (Q, K, P) walk the 128 bytes of a row in 32-byte k steps; the leading byte offset is unused.
// The MN-major operand (V: row = key = k index, 128 bytes = 64 channels of n) has its second 64-channel slab
// `lbo` bytes after the first and walks k in steps of 16 rows.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  return static_cast<uint64_t>((addr >> 4) & 0x3fffu) | (static_cast<uint64_t>((lbo >> 4) & 0x3fffu) << 16) |
         (static_cast<uint64_t>((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46) | (2ull << 61);
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
// attention
// ------------------------------------------------------------------------------------------------------
template <int D>
struct PfGeom {
  static constexpr int NSLAB = D / 64;                 // 64-channel slabs per operand tile
  static constexpr int Q_BYTES = NSLAB * PF_BM * 128;  // fp16 A operand of S = Q.K^T
  static constexpr int KV_SLAB = PF_BN * 128;          // one [64 keys][64 channels] fp16 slab
  static constexpr int KV_BYTES = NSLAB * KV_SLAB;
  static constexpr int P_BYTES = PF_BM * 128;          // [128 rows][64 keys] fp16
  static constexpr int STG_BYTES = PF_BN * D;          // int8 landing zone of one K or V step (four 16-key boxes)
  static constexpr int SMEM = 1024 + Q_BYTES + 2 * KV_BYTES + P_BYTES + 2 * STG_BYTES;
};

// int8 landing zone (TMA boxes of [16 keys][D bytes], hardware-swizzled) -> fp16 operand slabs. 16 channels per item.
template <int D>
__device__ __forceinline__ void widen_tile(const uint8_t* stg, uint8_t* dst, int tid) {
  constexpr int CPR = D / 16;   // 16-byte chunks per key row
#pragma unroll
  for (int i = 0; i < PF_BN * CPR / PF_THREADS; ++i) {
    const int idx = tid + PF_THREADS * i, key = idx / CPR, c = idx - key * CPR, kk = key & 15;
    const uint32_t src = (key >> 4) * 16 * D + kk * D + ((D == 128 ? (c ^ (kk & 7)) : (c ^ ((kk >> 1) & 3))) << 4);
    const uint4 w = *reinterpret_cast<const uint4*>(stg + src);
    uint4 lo, hi;
    i8x4_to_f16x4(w.x, lo.x, lo.y);
    i8x4_to_f16x4(w.y, lo.z, lo.w);
    i8x4_to_f16x4(w.z, hi.x, hi.y);
    i8x4_to_f16x4(w.w, hi.z, hi.w);
    uint8_t* slab = dst + (c >> 2) * PfGeom<D>::KV_SLAB;
    *reinterpret_cast<uint4*>(slab + slab_off(key, (c & 3) * 2)) = lo;
    *reinterpret_cast<uint4*>(slab + slab_off(key, (c & 3) * 2 + 1)) = hi;
  }
}

template <int D>
__global__ void __launch_bounds__(PF_THREADS, 2)
    prefill_kernel(const PrefillArgs a, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
  using Gm = PfGeom<D>;
  constexpr int NSLAB = Gm::NSLAB;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_bar[4];   // K landed, V landed, S = Q.K^T done, O += P.V done
  __shared__ uint32_t s_tmem;
  __shared__ int s_req;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_wait();   // the plan below is written by prefill_plan_kernel
  const int total = a.hdr[1];
  const int tix = blockIdx.x / a.Hkv, kvh = blockIdx.x - tix * a.Hkv;
  if (tix >= total) return;
  const int tile = total - 1 - tix;   // later m tiles of a request see more keys: start them first

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* p_base = smem_raw + (base - smem_u32(smem_raw));
  uint8_t* p_q = p_base;
  uint8_t* p_k = p_q + Gm::Q_BYTES;
  uint8_t* p_v = p_k + Gm::KV_BYTES;
  uint8_t* p_p = p_v + Gm::KV_BYTES;
  uint8_t* p_sk = p_p + Gm::P_BYTES;
  uint8_t* p_sv = p_sk + Gm::STG_BYTES;
  const uint32_t u_q = base, u_k = u_q + Gm::Q_BYTES, u_v = u_k + Gm::KV_BYTES, u_p = u_v + Gm::KV_BYTES,
                 u_sk = u_p + Gm::P_BYTES, u_sv = u_sk + Gm::STG_BYTES;
  const uint32_t bar_k = smem_u32(&s_bar[0]), bar_v = smem_u32(&s_bar[1]), bar_s = smem_u32(&s_bar[2]),
                 bar_o = smem_u32(&s_bar[3]);

  if (warp == 0) tmem_alloc(smem_u32(&s_tmem), PF_TMEM_COLS);
  if (tid == 0) {
    for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&s_bar[i]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int r = tid; r < a.num_seqs; r += PF_THREADS)
    if (a.prefix[r] <= tile && tile < a.prefix[r + 1]) s_req = r;
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem, t_s = tmem, t_o = tmem + PF_BN;
  const uint32_t t_lane = static_cast<uint32_t>(warp * 32) << 16;   // this warp's quarter of the 128 lanes

  const int req = s_req, mt = tile - a.prefix[req];
  const int tok0 = a.cu_q[req], qlen = a.cu_q[req + 1] - tok0, L = a.seq_lens[req];
  const int32_t* bt = a.block_table + static_cast<int64_t>(req) * a.bt_stride;
  const int t_first = mt * a.TQ, t_last = min(qlen, t_first + a.TQ) - 1;
  const int kmax = L - qlen + 1 + t_last;              // keys [0, kmax) are visible to the tile's last token
  const int nkt = kmax > 0 ? (kmax + PF_BN - 1) / PF_BN : 0;

  // ---- this thread's row ----
  const int tl = tid / a.G, hg = tid - tl * a.G, tq = t_first + tl;
  const bool valid = tl < a.TQ && tq < qlen;
  const int lim = valid ? L - qlen + 1 + tq : 0x7fffffff;   // padding rows hold q = 0 and are never stored
  float c_row = 0.f;
  {
    const __nv_bfloat16* qrow = a.q + static_cast<int64_t>(tok0 + tq) * a.q_st + static_cast<int64_t>(kvh * a.G + hg) * a.q_sh;
    const float* ksr = a.ks + kvh * (a.pc_k ? D : 1);
    float amax = 0.f;
    if (valid) {
#pragma unroll 4
      for (int c = 0; c < D / 8; ++c) {
        const uint4 w = __ldg(reinterpret_cast<const uint4*>(qrow) + c);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
        float s[8];
        if (a.pc_k) {
          const float4 s0 = __ldg(reinterpret_cast<const float4*>(ksr) + 2 * c), s1 = __ldg(reinterpret_cast<const float4*>(ksr) + 2 * c + 1);
          s[0] = s0.x, s[1] = s0.y, s[2] = s0.z, s[3] = s0.w, s[4] = s1.x, s[5] = s1.y, s[6] = s1.z, s[7] = s1.w;
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) s[e] = 1.f;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e)
          amax = fmaxf(amax, fmaxf(fabsf(bf16lo(ww[e]) * s[2 * e]), fabsf(bf16hi(ww[e]) * s[2 * e + 1])));
      }
    }
    // power-of-two row scale that puts the largest |q * s_k| into [2^14, 2^15): fp16 keeps 11 significant bits
    int ex = 0;
    if (amax > 0.f) frexpf(amax, &ex);
    const int sh = amax > 0.f ? max(-60, min(60, 15 - ex)) : 0;
    const float up = ldexpf(1.f, sh);
    c_row = a.scale_log2 * ldexpf(1.f, -sh) * (a.pc_k ? 1.f : __ldg(ksr));
#pragma unroll 2
    for (int c = 0; c < D / 8; ++c) {
      uint4 o = make_uint4(0u, 0u, 0u, 0u);
      if (valid) {
        const uint4 w = __ldg(reinterpret_cast<const uint4*>(qrow) + c);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
        float s[8];
        if (a.pc_k) {
          const float4 s0 = __ldg(reinterpret_cast<const float4*>(ksr) + 2 * c), s1 = __ldg(reinterpret_cast<const float4*>(ksr) + 2 * c + 1);
          s[0] = s0.x, s[1] = s0.y, s[2] = s0.z, s[3] = s0.w, s[4] = s1.x, s[5] = s1.y, s[6] = s1.z, s[7] = s1.w;
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) s[e] = 1.f;
        }
        uint32_t oo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) oo[e] = pack_f16x2(bf16lo(ww[e]) * s[2 * e] * up, bf16hi(ww[e]) * s[2 * e + 1] * up);
        o = make_uint4(oo[0], oo[1], oo[2], oo[3]);
      }
      *reinterpret_cast<uint4*>(p_q + (c >> 3) * (PF_BM * 128) + slab_off(tid, c & 7)) = o;
    }
  }

  // ---- TMA producer state (warp 0; lane i < 4 owns the i-th 16-key box of a step) ----
  auto page_of = [&](int j) {   // page id and offset of this lane's box of step j; boxes past the end re-read the first
    const int n0 = j * PF_BN, n = n0 + 16 * lane;
    return (n < L ? n : n0);
  };
  int pg_n = 0, pg_nn = 0;      // page ids of steps j + 1 and j + 2
  auto issue = [&](bool is_k, int j, int page) {
    const uint32_t bar = is_k ? bar_k : bar_v;
    if (lane == 0) mbar_expect_tx(bar, Gm::STG_BYTES);
    __syncwarp();
    if (lane < 4) {
      const int off = page_of(j) & a.bs_mask;
      const int* pos = is_k ? a.kpos : a.vpos;
      auto coord = [&](int s) { return pos[0] == s ? off : (pos[1] == s ? kvh : page); };
      tma_load_4d((is_k ? u_sk : u_sv) + lane * 16 * D, is_k ? &tm_k : &tm_v, 0, coord(1), coord(2), coord(3), bar);
    }
  };
  bool ok = true;
  int k_issued = 0, v_issued = 0, k_waited = 0, v_waited = 0, s_issued = 0, s_waited = 0, o_issued = 0, o_waited = 0;
  if (warp == 0 && nkt > 0) {
    int pg0 = 0;
    if (lane < 4) {
      pg0 = bt[page_of(0) >> a.lbs];
      if (nkt > 1) pg_n = bt[page_of(1) >> a.lbs];
    }
    issue(true, 0, pg0);
    issue(false, 0, pg0);
  }
  if (nkt > 0) k_issued = v_issued = 1;

  float m_ref = -1e30f, l_sum = 0.f;   // running maximum (log2 domain, held back) and denominator
  constexpr uint32_t ID_S = instr_desc(PF_BM, PF_BN, false), ID_O = instr_desc(PF_BM, D, true);

  for (int j = 0; j < nkt; ++j) {
    const uint32_t par = j & 1;
    if (warp == 0 && lane < 4 && j + 2 < nkt) pg_nn = bt[page_of(j + 2) >> a.lbs];
    // -- K of this step: widen, then S = Q.K^T on the tensor core --
    ok = ok && mbar_wait(bar_k, par);
    ++k_waited;
    if (ok) widen_tile<D>(p_sk, p_k, tid);
    fence_proxy_async();   // generic-proxy writes of the operand tiles (and of q before the first step) -> tensor core
    tc_fence_before();
    ok = __syncthreads_and(ok);
    if (!ok) break;
    if (warp == 0) {
      if (j + 1 < nkt) issue(true, j + 1, pg_n);
      if (lane == 0) {
        tc_fence_after();
#pragma unroll
        for (int sl = 0; sl < NSLAB; ++sl)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_f16(t_s, smem_desc(u_q + sl * (PF_BM * 128) + ks * 32, 16, 1024),
                     smem_desc(u_k + sl * Gm::KV_SLAB + ks * 32, 16, 1024), ID_S, (sl | ks) ? 1u : 0u);
        umma_commit(bar_s);
      }
    }
    if (j + 1 < nkt) ++k_issued;
    ++s_issued;
    // -- V of this step (the previous step's P.V must have finished reading the V and P tiles) --
    if (j > 0) {
      ok = ok && mbar_wait(bar_o, (j - 1) & 1);
      ++o_waited;
    }
    ok = ok && mbar_wait(bar_v, par);
    ++v_waited;
    if (ok) widen_tile<D>(p_sv, p_v, tid);
    // -- softmax of this thread's row --
    ok = ok && mbar_wait(bar_s, par);
    ++s_waited;
    tc_fence_after();
    if (__syncthreads_and(ok) == 0) {
      ok = false;
      break;
    }
    uint32_t sr[PF_BN];
    {
      uint32_t lo[32], hi[32];
      tmem_ld32(t_s + t_lane, lo);
      tmem_ld32(t_s + t_lane + 32, hi);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) sr[i] = lo[i], sr[32 + i] = hi[i];
    }
    const int n_base = j * PF_BN;
    float mx = -INFINITY;
    if (n_base + PF_BN <= lim) {
#pragma unroll
      for (int i = 0; i < PF_BN; ++i) mx = fmaxf(mx, __uint_as_float(sr[i]));
    } else {
#pragma unroll
      for (int i = 0; i < PF_BN; ++i) {
        if (n_base + i >= lim) sr[i] = 0xff800000u;   // -inf: exp2 gives exactly 0
        mx = fmaxf(mx, __uint_as_float(sr[i]));
      }
    }
    // scores are S * c_row with c_row > 0, so the row maximum of S gives the maximum score
    const float tile_max = mx * c_row;
    const bool grow = tile_max > m_ref + 8.f;
    float alpha = 1.f;
    if (grow) {
      alpha = ex2(m_ref - tile_max);   // 0 on the first step (m_ref = -1e30)
      m_ref = tile_max;
      l_sum *= alpha;
    }
    if (j > 0 && __any_sync(0xffffffffu, grow)) {   // rescale the accumulator rows of this warp in tensor memory
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t o[32];
        tmem_ld32(t_o + t_lane + c, o);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tmem_st32(t_o + t_lane + c, o);
      }
      tmem_wait_st();
    }
    {
      const float nm = -m_ref;
      float ls = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p0 = ex2(fmaf(__uint_as_float(sr[8 * c + 2 * e]), c_row, nm));
          const float p1 = ex2(fmaf(__uint_as_float(sr[8 * c + 2 * e + 1]), c_row, nm));
          ls += p0 + p1;
          w[e] = pack_f16x2(p0, p1);
        }
        *reinterpret_cast<uint4*>(p_p + slab_off(tid, c)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      l_sum += ls;
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
      if (j + 1 < nkt) issue(false, j + 1, pg_n);
      if (lane == 0) {
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_f16(t_o, smem_desc(u_p + ks * 32, 16, 1024), smem_desc(u_v + ks * 16 * 128, Gm::KV_SLAB, 1024), ID_O,
                   (j | ks) ? 1u : 0u);
        umma_commit(bar_o);
      }
      pg_n = pg_nn;
    }
    if (j + 1 < nkt) ++v_issued;
    ++o_issued;
  }

  // ---- epilogue: O / denominator * s_v -> bf16 ----
  if (ok && nkt > 0) {
    ok = mbar_wait(bar_o, (nkt - 1) & 1);
    ++o_waited;
    tc_fence_after();
  }
  ok = __syncthreads_and(ok);
  if (ok) {
    __nv_bfloat16* orow = a.out + static_cast<int64_t>(tok0 + tq) * a.o_st + static_cast<int64_t>(kvh * a.G + hg) * a.o_sh;
    const float inv = 1.f / fmaxf(l_sum, 1e-30f);
    const float* vsr = a.vs + kvh * (a.pc_v ? D : 1);
#pragma unroll 1
    for (int c = 0; c < D; c += 32) {
      uint32_t o[32];
      if (nkt > 0) {
        tmem_ld32(t_o + t_lane + c, o);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0u;
      }
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
  } else {
    // A bounded wait expired: report it, then give every copy and tensor-core operation that is still in flight
    // one more bounded chance to finish before shared and tensor memory are released.
    if (tid == 0) atomicExch(a.hdr, 1);
    if (k_issued > k_waited) mbar_wait(bar_k, k_waited & 1);
    if (v_issued > v_waited) mbar_wait(bar_v, v_waited & 1);
    if (s_issued > s_waited) mbar_wait(bar_s, s_waited & 1);
    if (o_issued > o_waited) mbar_wait(bar_o, o_waited & 1);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, PF_TMEM_COLS);
}

// ------------------------------------------------------------------------------------------------------
// warp-specialized variant: two m tiles per CTA share one K/V stream
// ------------------------------------------------------------------------------------------------------
// 13 warps: warps 0-3 and 4-7 are the softmax groups of m tile 0 and 1 (one thread per row), warps 8-11 widen the
// int8 K/V boxes into fp16 operand tiles and issue the TMA loads, warp 12 (one lane) issues every tcgen05.mma.
// The groups meet only through mbarriers, so S = Q.K^T of step j + 1 runs on the tensor core while the softmax
// groups work on step j, and O += P.V of step j starts the moment a group has written its P.
//   TMEM: S[tile][step & 1] 4 x 64 columns, O[tile] 2 x D columns.
//   smem: Q 2 tiles, fp16 K and V 2 stages each, P 2 buffers per tile, int8 landing zones 2 stages each.
constexpr int WS_THREADS = 13 * 32;
#ifdef KVQ_PF_TIMELINE
__device__ long long g_pf_timeline[3 * 64 * 8];   // [role][step][event]
#define PF_TL(role, step, ev)                                                                      \
  do {                                                                                             \
    if (blockIdx.x == gridDim.x / 2 && (step) < 64) g_pf_timeline[((role) * 64 + (step)) * 8 + (ev)] = clock64(); \
  } while (0)
#else
#define PF_TL(role, step, ev) do { } while (0)
#endif
constexpr int WS_TMEM_COLS = 512;
enum WsBar {
  WB_STGK = 0,       // [2] int8 K boxes landed (TMA)
  WB_STGV = 2,       // [2]
  WB_KF_READY = 4,   // [2] fp16 K tile written (128 converter threads)
  WB_VF_READY = 6,   // [2]
  WB_KF_FREE = 8,    // [2] tensor core done with the fp16 K tile (commit)
  WB_VF_FREE = 10,   // [2]
  WB_S_READY = 12,   // [tile * 2 + buffer] S computed (commit)
  WB_S_FREE = 16,    // [tile * 2 + buffer] S read into registers (128 softmax threads)
  WB_P_READY = 20,   // [tile * 2 + buffer] P written (128 softmax threads)
  WB_O_DONE = 24,    // [tile * 2 + (step & 1)] O += P.V of that step finished (commit)
  WB_Q_READY = 28,   // q tiles written (256 softmax threads)
  WB_STGK_FREE = 29, // [2] landing zone read by every converter (128 threads)
  WB_STGV_FREE = 31, // [2]
  WB_COUNT = 33
};

template <int D>
struct WsGeom {
  static constexpr int NSLAB = D / 64;
  static constexpr int Q_TILE = NSLAB * PF_BM * 128;
  static constexpr int KV_SLAB = PF_BN * 128;
  static constexpr int KV_TILE = NSLAB * KV_SLAB;
  static constexpr int P_TILE = PF_BM * 128;
  static constexpr int STG = PF_BN * D;
  static constexpr int OFF_Q = 0, OFF_K = OFF_Q + 2 * Q_TILE, OFF_V = OFF_K + 2 * KV_TILE, OFF_P = OFF_V + 2 * KV_TILE,
                       OFF_SK = OFF_P + 4 * P_TILE, OFF_SV = OFF_SK + 2 * STG, END = OFF_SV + 2 * STG;
  static constexpr int SMEM = 1024 + END;
};

// Bounded wait that also gives up as soon as any thread of the CTA has given up. Called by converged warps; the
// result is uniform over the warp, so the warp-collective tensor-memory instructions that follow stay converged.
__device__ __forceinline__ bool ws_wait_thread(uint32_t bar, uint32_t parity, volatile int* abort_flag);
__device__ __forceinline__ bool ws_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, ws_wait_thread(bar, parity, abort_flag));
}
__device__ __forceinline__ bool ws_wait_thread(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > (1ll << 31)) {
      *abort_flag = 1;
      return false;
    }
  }
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
      const int n = (i >= WB_KF_READY && i < WB_KF_FREE) || (i >= WB_S_FREE && i < WB_O_DONE) || i >= WB_STGK_FREE
                        ? 128
                        : (i == WB_Q_READY ? 256 : 1);
      mbar_init(bar(i), n);
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
    return kmax > 0 ? (kmax + PF_BN - 1) / PF_BN : 0;
  };
  const int nk0 = steps_of(mt0), nk1 = steps_of(mt0 + 1), nk = max(nk0, nk1);
  constexpr uint32_t ID_S = instr_desc(PF_BM, PF_BN, false), ID_O = instr_desc(PF_BM, D, true);

  if (warp < 8) {
    // ================= softmax group of m tile t =================
    const int t = warp >> 2, row = tid & 127, mt = mt0 + t, nkt = t ? nk1 : nk0;
    uint8_t* p_q = p_base + Gm::OFF_Q + t * Gm::Q_TILE;
    uint8_t* p_p = p_base + Gm::OFF_P + t * 2 * Gm::P_TILE;   // two buffers, by step parity
    const uint32_t t_lane = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem + t * 2 * PF_BN + t_lane, t_o = tmem + 4 * PF_BN + t * D + t_lane;
    const int tl = row / a.G, hg = row - tl * a.G, tq = mt * a.TQ + tl;
    const bool valid = tl < a.TQ && tq < qlen;
    const int lim = valid ? L - qlen + 1 + tq : 0x7fffffff;   // padding rows hold q = 0 and are never stored
    float c_row = 0.f;
    {
      const __nv_bfloat16* qrow = a.q + static_cast<int64_t>(tok0 + tq) * a.q_st + static_cast<int64_t>(kvh * a.G + hg) * a.q_sh;
      const float* ksr = a.ks + kvh * (a.pc_k ? D : 1);
      auto scaled = [&](int c, float (&f)[8]) {   // channels 8c..8c+7 of q * s_k
        const uint4 w = __ldg(reinterpret_cast<const uint4*>(qrow) + c);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) f[2 * e] = bf16lo(ww[e]), f[2 * e + 1] = bf16hi(ww[e]);
        if (a.pc_k) {
          const float4 s0 = __ldg(reinterpret_cast<const float4*>(ksr) + 2 * c), s1 = __ldg(reinterpret_cast<const float4*>(ksr) + 2 * c + 1);
          f[0] *= s0.x, f[1] *= s0.y, f[2] *= s0.z, f[3] *= s0.w, f[4] *= s1.x, f[5] *= s1.y, f[6] *= s1.z, f[7] *= s1.w;
        }
      };
      float amax = 0.f;
      if (valid) {
#pragma unroll 4
        for (int c = 0; c < D / 8; ++c) {
          float f[8];
          scaled(c, f);
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
#pragma unroll 2
      for (int c = 0; c < D / 8; ++c) {
        uint4 o = make_uint4(0u, 0u, 0u, 0u);
        if (valid) {
          float f[8];
          scaled(c, f);
          o = make_uint4(pack_f16x2(f[0] * up, f[1] * up), pack_f16x2(f[2] * up, f[3] * up), pack_f16x2(f[4] * up, f[5] * up),
                         pack_f16x2(f[6] * up, f[7] * up));
        }
        *reinterpret_cast<uint4*>(p_q + (c >> 3) * (PF_BM * 128) + slab_off(row, c & 7)) = o;
      }
    }
    fence_proxy_async();
    mbar_arrive(bar(WB_Q_READY));

    float m_ref = -1e30f, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < nkt && ok; ++j) {
      const int b = j & 1;
      if (tid == 0) PF_TL(0, j, 0);
      ok = ws_wait(bar(WB_S_READY + t * 2 + b), (j >> 1) & 1, abort_flag);
      if (!ok) break;
      if (tid == 0) PF_TL(0, j, 1);
      tc_fence_after();
      uint32_t sr[PF_BN];
      {
        uint32_t lo[32], hi[32];
        tmem_ld32(t_s + b * PF_BN, lo);
        tmem_ld32(t_s + b * PF_BN + 32, hi);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) sr[i] = lo[i], sr[32 + i] = hi[i];
      }
      tc_fence_before();
      if (tid == 0) PF_TL(0, j, 2);
      mbar_arrive(bar(WB_S_FREE + t * 2 + b));
      if (tid == 0) PF_TL(0, j, 3);
      const int n_base = j * PF_BN;
      float mx = -INFINITY;
      if (n_base + PF_BN <= lim) {
#pragma unroll
        for (int i = 0; i < PF_BN; ++i) mx = fmaxf(mx, __uint_as_float(sr[i]));
      } else {
#pragma unroll
        for (int i = 0; i < PF_BN; ++i) {
          if (n_base + i >= lim) sr[i] = 0xff800000u;   // -inf: exp2 gives exactly 0
          mx = fmaxf(mx, __uint_as_float(sr[i]));
        }
      }
      const float tile_max = mx * c_row;   // c_row > 0
      const bool grow = tile_max > m_ref + 8.f;
      float alpha = 1.f;
      if (grow) {
        alpha = ex2(m_ref - tile_max);   // 0 on the first step (m_ref = -1e30)
        m_ref = tile_max;
        l_sum *= alpha;
      }
      if (tid == 0) PF_TL(0, j, 4);
      if (j >= 2) {   // P.V of step j - 2 has finished reading this step's P buffer
        ok = ws_wait(bar(WB_O_DONE + t * 2 + b), ((j - 2) >> 1) & 1, abort_flag);
        if (!ok) break;
      }
      if (j > 0 && __any_sync(0xffffffffu, grow)) {   // rescale O (rare after the first steps): P.V of step j - 1 first
        ok = ws_wait(bar(WB_O_DONE + t * 2 + (b ^ 1)), ((j - 1) >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        {
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t o[32];
            tmem_ld32(t_o + c, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(t_o + c, o);
          }
          tmem_wait_st();
        }
      }
      if (tid == 0) PF_TL(0, j, 5);
      {
        const float nm = -m_ref;
        float ls = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float p0 = ex2(fmaf(__uint_as_float(sr[8 * c + 2 * e]), c_row, nm));
            const float p1 = ex2(fmaf(__uint_as_float(sr[8 * c + 2 * e + 1]), c_row, nm));
            ls += p0 + p1;
            w[e] = pack_f16x2(p0, p1);
          }
          *reinterpret_cast<uint4*>(p_p + b * Gm::P_TILE + slab_off(row, c)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        l_sum += ls;
      }
      if (tid == 0) PF_TL(0, j, 6);
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(bar(WB_P_READY + t * 2 + b));
      if (tid == 0) PF_TL(0, j, 7);
    }
    // ---- epilogue: O / denominator * s_v -> bf16 ----
    if (ok && nkt > 0) ok = ws_wait(bar(WB_O_DONE + t * 2 + ((nkt - 1) & 1)), ((nkt - 1) >> 1) & 1, abort_flag);
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
    // ================= converters: TMA issue + int8 -> fp16 =================
    const int ctid = tid - 256;
    const bool issuer = warp == 8;
    auto key_of = [&](int j) {   // first key of this lane's 16-key box of step j; boxes past the end re-read the first
      const int n0 = j * PF_BN, n = n0 + 16 * lane;
      return n < L ? n : n0;
    };
    auto issue = [&](bool is_k, int j, int page) {   // warp 8: lane i < 4 loads the i-th box
      const uint32_t full = bar((is_k ? WB_STGK : WB_STGV) + (j & 1));
      if (lane == 0) mbar_expect_tx(full, Gm::STG);
      __syncwarp();
      if (lane < 4) {
        const int off = key_of(j) & a.bs_mask;
        const int* pos = is_k ? a.kpos : a.vpos;
        auto coord = [&](int s) { return pos[0] == s ? off : (pos[1] == s ? kvh : page); };
        tma_load_4d(base + (is_k ? Gm::OFF_SK : Gm::OFF_SV) + (j & 1) * Gm::STG + lane * 16 * D, is_k ? &tm_k : &tm_v, 0,
                    coord(1), coord(2), coord(3), full);
      }
    };
    int pg_a = 0, pg_b = 0;   // page ids (lanes 0-3 of warp 8) of the next two steps to issue
    if (issuer) {
      if (lane < 4) {
        if (nk > 0) pg_a = bt[key_of(0) >> a.lbs];
        if (nk > 1) pg_b = bt[key_of(1) >> a.lbs];
      }
      if (nk > 0) issue(true, 0, pg_a), issue(false, 0, pg_a);
      if (nk > 1) issue(true, 1, pg_b), issue(false, 1, pg_b);
      pg_a = 0, pg_b = 0;
      if (lane < 4) {
        if (nk > 2) pg_a = bt[key_of(2) >> a.lbs];
        if (nk > 3) pg_b = bt[key_of(3) >> a.lbs];
      }
    }
    bool ok = true;
    for (int j = 0; j < nk && ok; ++j) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      // pg_a belongs to step j + 2 (issued below), pg_b to step j + 3
      if (ctid == 0) PF_TL(1, j, 0);
      ok = ws_wait(bar(WB_STGK + s), ph, abort_flag);
      if (ctid == 0) PF_TL(1, j, 1);
      if (ok && j >= 2) ok = ws_wait(bar(WB_KF_FREE + s), ((j - 2) >> 1) & 1, abort_flag);
      if (!ok) break;
      if (ctid == 0) PF_TL(1, j, 2);
      widen_tile<D>(p_base + Gm::OFF_SK + s * Gm::STG, p_base + Gm::OFF_K + s * Gm::KV_TILE, ctid);
      fence_proxy_async();
      mbar_arrive(bar(WB_KF_READY + s));
      mbar_arrive(bar(WB_STGK_FREE + s));
      if (ctid == 0) PF_TL(1, j, 3);
      if (issuer && j + 2 < nk) {   // every converter has left the landing zone before it is refilled
        ok = ws_wait(bar(WB_STGK_FREE + s), ph, abort_flag);
        if (ok) issue(true, j + 2, pg_a);
      }
      if (ctid == 0) PF_TL(1, j, 4);
      ok = ws_wait(bar(WB_STGV + s), ph, abort_flag);
      if (ctid == 0) PF_TL(1, j, 5);
      if (ok && j >= 2) ok = ws_wait(bar(WB_VF_FREE + s), ((j - 2) >> 1) & 1, abort_flag);
      if (!ok) break;
      if (ctid == 0) PF_TL(1, j, 6);
      widen_tile<D>(p_base + Gm::OFF_SV + s * Gm::STG, p_base + Gm::OFF_V + s * Gm::KV_TILE, ctid);
      fence_proxy_async();
      mbar_arrive(bar(WB_VF_READY + s));
      mbar_arrive(bar(WB_STGV_FREE + s));
      if (ctid == 0) PF_TL(1, j, 7);
      if (issuer) {
        if (j + 2 < nk) {
          ok = ok && ws_wait(bar(WB_STGV_FREE + s), ph, abort_flag);
          if (ok) issue(false, j + 2, pg_a);
        }
        pg_a = pg_b;
        pg_b = (lane < 4 && j + 4 < nk) ? bt[key_of(j + 4) >> a.lbs] : 0;
      }
    }
  } else if (lane == 0) {
    // ================= tensor-core issue (one thread) =================
    bool ok = ws_wait_thread(bar(WB_Q_READY), 0, abort_flag);
    // Descriptors differ only in their 14-bit start-address field (address >> 4): one base per operand, the
    // tile / slab / k-step offsets (compile-time constants once the loops are unrolled) are added to it.
    const uint64_t d_q = smem_desc(base + Gm::OFF_Q, 16, 1024), d_k = smem_desc(base + Gm::OFF_K, 16, 1024),
                   d_p = smem_desc(base + Gm::OFF_P, 16, 1024), d_v = smem_desc(base + Gm::OFF_V, Gm::KV_SLAB, 1024);
    auto issue_qk = [&](int j) {
      const int s = j & 1;
      ok = ok && ws_wait_thread(bar(WB_KF_READY + s), (j >> 1) & 1, abort_flag);
      const uint64_t d_ks = d_k + static_cast<uint64_t>((s * Gm::KV_TILE) >> 4);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (!ok || j >= (t ? nk1 : nk0)) continue;
        if (j >= 2) ok = ws_wait_thread(bar(WB_S_FREE + t * 2 + s), ((j - 2) >> 1) & 1, abort_flag);
        if (!ok) continue;
        tc_fence_after();
        const uint32_t d_s = tmem + (t * 2 + s) * PF_BN;
#pragma unroll
        for (int sl = 0; sl < NSLAB; ++sl)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_f16(d_s, d_q + static_cast<uint64_t>((t * Gm::Q_TILE + sl * (PF_BM * 128) + ks * 32) >> 4),
                     d_ks + static_cast<uint64_t>((sl * Gm::KV_SLAB + ks * 32) >> 4), ID_S, (sl | ks) ? 1u : 0u);
        umma_commit(bar(WB_S_READY + t * 2 + s));
      }
      if (ok) umma_commit(bar(WB_KF_FREE + s));
    };
    if (ok && nk > 0) issue_qk(0);
    for (int j = 0; j < nk && ok; ++j) {
      const int s = j & 1;
      PF_TL(2, j, 0);
      if (j + 1 < nk) issue_qk(j + 1);
      PF_TL(2, j, 1);
      ok = ok && ws_wait_thread(bar(WB_VF_READY + s), (j >> 1) & 1, abort_flag);
      PF_TL(2, j, 2);
      const uint64_t d_vs = d_v + static_cast<uint64_t>((s * Gm::KV_TILE) >> 4);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (!ok || j >= (t ? nk1 : nk0)) continue;
        ok = ws_wait_thread(bar(WB_P_READY + t * 2 + s), (j >> 1) & 1, abort_flag);
        if (!ok) continue;
        tc_fence_after();
        const uint64_t d_ps = d_p + static_cast<uint64_t>(((t * 2 + s) * Gm::P_TILE) >> 4);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_f16(tmem + 4 * PF_BN + t * D, d_ps + static_cast<uint64_t>((ks * 32) >> 4),
                   d_vs + static_cast<uint64_t>((ks * 16 * 128) >> 4), ID_O, (j | ks) ? 1u : 0u);
        umma_commit(bar(WB_O_DONE + t * 2 + s));
        PF_TL(2, j, 3 + t);
      }
      if (ok) umma_commit(bar(WB_VF_FREE + s));
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
    KVQ_CUDA(cudaFuncSetAttribute(prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, PfGeom<64>::SMEM));
    KVQ_CUDA(cudaFuncSetAttribute(prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, PfGeom<128>::SMEM));
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

  // KVQ_PREFILL_SIMPLE=1 selects the one-m-tile-per-CTA kernel without warp specialization (debugging aid)
  static const bool simple = [] {
    const char* e = getenv("KVQ_PREFILL_SIMPLE");
    return e && e[0] == '1';
  }();
  const int per_cta = simple ? 1 : 2;
  prefill_plan_kernel<<<1, 256, 0, s>>>(cu_q, num_seqs, a.TQ, a.min_q, per_cta, a.hdr, a.prefix);
  KVQ_CUDA(cudaGetLastError());
  // upper bound of the work items: sum over requests of ceil(m tiles / per_cta), m tiles = ceil(q_len / TQ)
  const int64_t max_items = total_query_tokens / (static_cast<int64_t>(a.TQ) * per_cta) + num_seqs;
  KVQ_REQUIRE(max_items * num_kv_heads < (1ll << 31), "prefill_attention: batch too large");
  const dim3 grid(static_cast<unsigned>(max_items * num_kv_heads));
  if (simple) {
    if (head_dim == 128)
      KVQ_CUDA(pf_launch_pdl(prefill_kernel<128>, grid, dim3(PF_THREADS), PfGeom<128>::SMEM, s, a, tm_k, tm_v));
    else
      KVQ_CUDA(pf_launch_pdl(prefill_kernel<64>, grid, dim3(PF_THREADS), PfGeom<64>::SMEM, s, a, tm_k, tm_v));
  } else {
    if (head_dim == 128)
      KVQ_CUDA(pf_launch_pdl(prefill_ws_kernel<128>, grid, dim3(WS_THREADS), WsGeom<128>::SMEM, s, a, tm_k, tm_v));
    else
      KVQ_CUDA(pf_launch_pdl(prefill_ws_kernel<64>, grid, dim3(WS_THREADS), WsGeom<64>::SMEM, s, a, tm_k, tm_v));
  }
  return KVQ_OK;
}

#ifdef KVQ_PF_TIMELINE
extern "C" __attribute__((visibility("default"))) int kvq_debug_pf_timeline(long long* host, int n) {
  return cudaMemcpyFromSymbol(host, g_pf_timeline, sizeof(long long) * n) == cudaSuccess ? 0 : 1;
}
#endif
