// INT8 paged attention for short queries (decode and speculative-decoding verification) on sm_100a.
//
// Two launches per call (three for batches of more than FUSED_PLAN_MAX requests), all on the caller's stream, no host
// synchronization:
//   decode_kernel   one CTA per slice of the global unit range (a unit is one 32-key chunk of one item; the range is
//                   cut into equal shares of a cost, one per unit plus a figure per item start, over #SMs x resident
//                   CTAs, so every CTA streams nearly the same number of KV bytes whatever the mix of context lengths
//                   and short ranges do not cross item boundaries); a slice covers whole (request, kv head, m-tile group) items and at
//                   most two partial ones, whose (acc, max, sum) go to the workspace. Every CTA sums the per-request
//                   work itself to find its slice (a block scan over the requests instead of a kernel boundary)
//   merge_kernel    items that were cut across CTAs: combine their partials into the output; folds the CTAs' status
//   plan_kernel     large batches only, first: per-request units and costs, their exclusive prefix sums in the workspace, so
//                   that hundreds of CTAs do not each walk thousands of requests
//
// Inside decode_kernel the four warps of a CTA form groups of 1, 2 or 4 (per request, by its number of 16-row
// m tiles). A group owns a slice of the TMA ring (cp.async.bulk.tensor, 128-byte swizzle, one 16-key x head_dim
// box per page half, full/empty mbarriers) and streams its own 32-key chunks; every warp of the group reads
// the same stage and works on its own m tile: S = Q.K^T with mma.sync m16n8k32 s8 (K fragments by ldmatrix),
// fp32 online softmax, P quantized to int8 per (row, chunk), O += P.V with the same mma (V fragments by the
// 8-bit transposing ldmatrix of sm_100). Warps that worked on the same m tile are combined through shared memory.
//
// Numerics follow "implementation B" of the reference (kvq/int8_ref.py:108-143, kernel restatement
// kvq/cuda/int8_kv.cu:11-15): see include/kvq_b200.h.
#include <cstdlib>
#include <type_traits>
#include <cuda.h>

#include <mutex>
#include <vector>

#include "kvq_common.cuh"
#include "kvq_host.h"
#include "kvq_ptx.cuh"

namespace kvq {
namespace {

constexpr int CHUNK = 32;      // keys per pipeline stage and per P-quantization tile
constexpr int NWARPS = 4;
constexpr int NTHREADS = NWARPS * 32;
constexpr int FUSED_PLAN_MAX = 1024;  // up to this many requests every CTA sums the work itself; beyond, plan_kernel runs first
constexpr int MIN_UNITS = 4;   // never give a CTA less than one chunk per warp
constexpr int MAX_CTAS_PER_SM = 4;
constexpr int HDR_BYTES = 256;  // workspace header: int32 [0] status, [1] total units, [2] cost share per CTA, [3] total cost
constexpr int PART_ROWS = 16;      // rows of one m tile
constexpr int PART_ROWS_GROUPED = 64;  // rows of a group of up to four m tiles

struct DecodeArgs {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  const int32_t *cu_q, *seq_lens, *block_table;
  const float *ks, *vs;
  int32_t* hdr;
  const int32_t* prefix;   // [2][num_seqs + 1] exclusive prefixes of per-request units and costs (only when planned)
  int32_t* cta_status;     // [grid] 1 where a bounded wait of that CTA expired (folded into hdr[0] by the merge kernel)
  int32_t* bnd;            // [grid][8] what the end of each CTA's range cut (written by decode, read by merge)
  float* part_acc;         // [grid * 2][16][D]  numerator * v_scale of a cut item
  float* part_ml;          // [grid * 2][16][2]  running max of the scores, denominator
  float sm_hi, sm_lo;      // softmax scale (natural-log domain) as an unevaluated fp32 pair
  int num_seqs, Hq, Hkv, G, lbs, bs_mask, qmax;
  int64_t q_st, q_sh, o_st, o_sh, bt_stride;
  int pc_k, pc_v;
  int planned;             // 1: plan_kernel ran first (large batches); 0: every CTA derives its slice itself
  int grouped;             // 1: warps of a CTA share K/V streams across m tiles (multi-token queries)
  int hg;                  // 0, or 2 / 4: decode with warps of a group on ADJACENT KV HEADS of one stream (see req_shape)
  int part_rows;           // rows per partial slot: 16, or 64 in grouped mode
  int item_cost;           // what starting an item costs a CTA, in units (see work_cost)
  int kpos[3], vpos[3];    // tensor-map coordinate slot (1..3) of the (slot-in-block, head, block) dims
};

// ------------------------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// Two 16x16 byte matrices, transposed: with lane l pointing at row l of a [32 keys][16 channels] block, lane
// (g = l / 4, t = l % 4) receives r0 = rows 4t..4t+3 of column g, r1 = same rows of column g + 8, and r2, r3
// the same for rows 16 + 4t.. : the B fragments (k = keys, n = channels) of two m16n8k32 tiles.
__device__ __forceinline__ void ldsm_t8_x2(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m16n16.x2.trans.shared.b8 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Same with a zero accumulator input: the instruction takes the zero register, so nothing has to be cleared first.
__device__ __forceinline__ void mma_s8_zero(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}

// Unevaluated sum hi + lo of two floats (|lo| <= ulp(hi) / 2): ~48 bits of significand without FP64 instructions.
struct ff {
  float hi, lo;
};
__device__ __forceinline__ ff fast_two_sum(float a, float b) {  // |a| >= |b|
  const float s = __fadd_rn(a, b);
  return ff{s, __fadd_rn(b, -__fadd_rn(s, -a))};
}
__device__ __forceinline__ ff two_prod(float a, float b) {
  const float p = __fmul_rn(a, b);
  return ff{p, __fmaf_rn(a, b, -p)};
}
__device__ __forceinline__ ff ff_mul(ff a, ff b) {
  const float p = __fmul_rn(a.hi, b.hi);
  float e = __fmaf_rn(a.hi, b.hi, -p);
  e = __fmaf_rn(a.hi, b.lo, e);
  e = __fmaf_rn(a.lo, b.hi, e);
  return fast_two_sum(p, e);
}
__device__ __forceinline__ ff ff_max(ff a, ff b) { return (b.hi > a.hi || (b.hi == a.hi && b.lo > a.lo)) ? b : a; }

// Byte offset of (key row tau, 16-byte column c16) inside a TMA-written tile of D-byte rows. The tile base
// is 1024-byte aligned; TMA's 128B swizzle XORs address bits [4:6] with bits [7:9] (64B: bits [4:5] with [7:8]).
// A tile is two TMA boxes of 16 keys; a box holds hs heads per key ([key][head][D], hs = 1 except in head-group
// mode) and this warp reads head hsel of it.
template <int D>
__device__ __forceinline__ uint32_t tile_off(int tau, int c16, int hs = 1, int hsel = 0) {
  const uint32_t off = ((tau >> 4) * 16 * hs + (tau & 15) * hs + hsel) * D + c16 * 16;
  return off ^ (((off >> 7) & (D == 128 ? 7u : 3u)) << 4);
}

// Work of one request. A request with q_len query tokens has ceil(q_len * G / 16) m tiles of 16 (token, head) rows
// per kv head. Units are 32-key chunks of items; what an item is depends on the mode:
//   plain      (kv head, m tile)
//   grouped    (kv head, group of gs m tiles): gs warps share one K/V stream and take one m tile each
//   hg = 2, 4  (group of hg adjacent kv heads), decode only: one stream carries the K/V rows of hg heads (a token's
//              heads are contiguous in a token-major cache, so every TMA box reads hg x head_dim contiguous bytes per
//              key instead of head_dim) and each of the gs = hg warps takes one head
struct ReqShape {
  int nchunks, mtiles, gs, mgroups, units, items;   // units = items * nchunks
};
__host__ __device__ __forceinline__ ReqShape req_shape(int qlen, int L, int G, int Hkv, int qmax, int grouped, int hg) {
  ReqShape r;
  r.nchunks = max(1, (L + CHUNK - 1) / CHUNK);
  r.mtiles = (qlen * G + 15) / 16;
  if (hg) {
    r.gs = hg, r.mgroups = 1;
    r.items = (qlen < 1 || qlen > qmax) ? 0 : Hkv / hg;
    r.units = r.items * r.nchunks;
    return r;
  }
  r.gs = grouped ? (r.mtiles >= 3 ? 4 : (r.mtiles == 2 ? 2 : 1)) : 1;
  r.mgroups = (r.mtiles + r.gs - 1) / r.gs;
  r.items = (qlen < 1 || qlen > qmax) ? 0 : Hkv * r.mgroups;
  r.units = r.items * r.nchunks;
  return r;
}

// The CTAs do not split the units evenly but a cost: one per unit plus `item_cost` per item start. Starting an item in
// the middle of a CTA's range drains its TMA ring, combines the warps, writes the item out and runs the next q prologue
// (~5 us, measured), so a CTA whose range crosses an item boundary used to finish that much after the others: at small
// batches (a few long requests over all SMs) those few CTAs set the kernel's time. In cost space an item is a jump of
// item_cost followed by its units; ranges are equal in cost, and a range boundary that falls inside a jump snaps to the
// item's first unit, so short ranges stop crossing item boundaries at all.
__host__ __device__ __forceinline__ int work_cost(const ReqShape& r, int item_cost) { return r.units + item_cost * r.items; }
// Unit (relative to the request's first) at cost f (relative to the request's first): the inverse of the cost function.
__host__ __device__ __forceinline__ int unit_at_cost(const ReqShape& r, int item_cost, int f) {
  const int per = r.nchunks + item_cost, item = f / per, o = f - item * per;
  return item * r.nchunks + max(0, o - item_cost);
}

// ------------------------------------------------------------------------------------------------------
// plan: units and cost per request, exclusive prefix sums, cost share per CTA
// ------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) plan_kernel(const int32_t* __restrict__ cu_q, const int32_t* __restrict__ seq_lens,
                                                   int num_seqs, int G, int Hkv, int qmax, int grouped, int hg, int item_cost,
                                                   int nctas, int32_t* __restrict__ hdr, int32_t* __restrict__ prefix) {
  __shared__ unsigned long long s_warp[8];
  __shared__ unsigned long long s_carry;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int32_t* prefix_f = prefix + num_seqs + 1;
  pdl_launch_dependents();   // the attention kernel may set itself up while the plan is computed
  if (tid == 0) s_carry = 0;
  __syncthreads();
  for (int base = 0; base < num_seqs; base += 256) {
    const int r = base + tid;
    unsigned long long u = 0;   // cost in the high word, units in the low word
    if (r < num_seqs) {
      const ReqShape rs = req_shape(cu_q[r + 1] - cu_q[r], seq_lens[r], G, Hkv, qmax, grouped, hg);
      u = (static_cast<unsigned long long>(work_cost(rs, item_cost)) << 32) | static_cast<unsigned>(rs.units);
    }
    unsigned long long x = u;  // inclusive scan inside the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) s_warp[warp] = x;
    __syncthreads();
    unsigned long long woff = 0;
    for (int w = 0; w < warp; ++w) woff += s_warp[w];
    const unsigned long long carry = s_carry, excl = carry + woff + x - u;
    if (r < num_seqs) prefix[r] = static_cast<int>(excl & 0xffffffffu), prefix_f[r] = static_cast<int>(excl >> 32);
    __syncthreads();
    if (tid == 255) s_carry = carry + woff + x;
    __syncthreads();
  }
  if (tid == 0) {
    const int total = static_cast<int>(s_carry & 0xffffffffu), total_f = static_cast<int>(s_carry >> 32);
    prefix[num_seqs] = total, prefix_f[num_seqs] = total_f;
    hdr[1] = total;
    hdr[2] = max((total_f + nctas - 1) / nctas, MIN_UNITS);
    hdr[3] = total_f;
  }
}

// ------------------------------------------------------------------------------------------------------
// main kernel
// ------------------------------------------------------------------------------------------------------
// Warps of a CTA are organised in groups of GS warps (GS = 1, 2 or 4, chosen per request from its number of
// 16-row m tiles). A group streams its own 32-key chunks through its own slice of the TMA ring; inside a group
// every warp reads the same K/V stage from shared memory and works on its own m tile, so K/V bytes are fetched
// from HBM once however many query rows use them. GS = 1 (decode: all rows of a kv head fit one m tile) gives
// four independent streams per CTA; GS = 4 (e.g. 8 query tokens x 7 heads = 56 rows) gives one stream feeding
// four m tiles. Groups that worked on the same m tile are combined through shared memory at the end of an item.
template <int D, bool ROWS16>
struct Geom {
  // The 16-row variant (multi-token queries) is bound by its instruction stream at two register-limited warps per
  // scheduler, not by HBM: it runs three CTAs per SM (168 registers per thread) on a ring of two stages per warp,
  // which keeps the same number of bytes in flight per SM as the 8-row decode variant's two CTAs of three stages.
  static constexpr int NSTAGE = ROWS16 ? 2 : 3;   // TMA ring depth per warp
  static constexpr int MIN_CTAS = ROWS16 ? 3 : 2; // resident CTAs per SM the kernel is compiled for
  static constexpr int TILE = CHUNK * D;          // one K or V chunk
  static constexpr int STAGE = 2 * TILE;          // K chunk + V chunk
  static constexpr int NSTG = NWARPS * NSTAGE;    // stages per CTA
  static constexpr int RING = NSTG * STAGE;
  static constexpr int SLOTS = NWARPS;            // m tiles (or kv heads of a head group) a CTA holds q for
  static constexpr int QROW = D;                  // s_q row stride (read once per item: bank conflicts do not matter)
  static constexpr int ACC_RS = D + 8;            // combine buffer row stride in floats
  static constexpr int SMALL = SLOTS * 16 * QROW + 6 * 64 * 4;
  static constexpr int SMEM = 1024 + RING + SMALL;  // 1024: manual alignment of the ring
  static_assert(NWARPS * 16 * ACC_RS * 4 <= RING, "combine buffer aliases the ring");
};

// One row of q (4 channels per lane): exact fold of s_k, row scale, int8 row into s_q, score scale into
// s_chi / s_clo. Called by a full warp. The reference's implementation B does this in double (exact products
// q * s_k, scale = max / 127, division). FP64 issue is slow on this part, so the same values are carried as
// unevaluated fp32 pairs (~2^-46); only exact rounding ties take the literal double route.
//
// QG: one q scale per 32 channels instead of one per row (the reference's q_gran="group32", kvq/int8_ref.py:120-130):
// the maximum is taken over the 8 lanes of a slice, and the slice's score scale (fp32) goes to s_chi[row * D / 32 + slice].
template <int D, bool QG = false>
__device__ __forceinline__ void q_quantize_row(const DecodeArgs& a, uint2 raw, const float (&sk)[4], int8_t* s_q,
                                               float* s_chi, float* s_clo, int kvh, int row, int lane) {
  constexpr int QROW = D, LANES = D / 4;
  const bool lane_on = lane < LANES;
  const int d0 = (lane_on ? lane : 0) * 4;
  float x[4] = {bf16lo(raw.x), bf16hi(raw.x), bf16lo(raw.y), bf16hi(raw.y)};
  ff amax = {0.f, 0.f};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const ff p = two_prod(x[e], sk[e]);   // exact product as hi + lo
    x[e] = p.hi;                          // fp32(q * s_k): what gets quantized
    amax = ff_max(amax, ff{fabsf(p.hi), p.hi < 0.f ? -p.lo : p.lo});
  }
#pragma unroll
  for (int o = 1; o < (QG ? 8 : 32); o <<= 1)
    amax = ff_max(amax, ff{__shfl_xor_sync(0xffffffffu, amax.hi, o), __shfl_xor_sync(0xffffffffu, amax.lo, o)});
  // sq = max(amax / 127, 1e-8)
  ff sq;
  {
    const float q1 = __fdiv_rn(amax.hi, 127.f);
    const float rem = __fmaf_rn(-q1, 127.f, amax.hi);            // exact remainder of the rounded quotient
    sq = fast_two_sum(q1, __fdiv_rn(__fadd_rn(rem, amax.lo), 127.f));
    constexpr float E_HI = 1e-8f;
    const float E_LO = static_cast<float>(1e-8 - static_cast<double>(E_HI));   // folded at compile time
    if (sq.hi < E_HI || (sq.hi == E_HI && sq.lo < E_LO)) sq = ff{E_HI, E_LO};
  }
  int b[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    // rint(x / sq): the fp32 quotient is within 2e-5 of the exact one (|quotient| <= 127). Only a value that
    // close to k + 0.5 takes the reference's literal double-precision route (exact ties do occur with a
    // per-head K scale, where x / sq is a ratio of bf16 numbers, and there the double roundings decide).
    const float qf = __fdiv_rn(x[e], sq.hi);
    int r = __float2int_rn(qf);
    if (fabsf(fabsf(qf - static_cast<float>(r)) - 0.5f) < 1e-4f) {
      const double sqd = fmax((static_cast<double>(amax.hi) + static_cast<double>(amax.lo)) / 127.0, 1e-8);
      r = __double2int_rn(static_cast<double>(x[e]) / sqd);
    }
    b[e] = max(-127, min(127, r));
  }
  if (lane_on) *reinterpret_cast<uint32_t*>(&s_q[row * QROW + d0]) = pack4(b[0], b[1], b[2], b[3]);
  if (QG ? ((lane & 7) == 0 && lane_on) : lane == 0) {
    // score = int32 dot * c, c = s_q [* s_k per head] * softmax_scale kept as an unevaluated hi + lo pair
    ff c = sq;
    if (!a.pc_k) c = ff_mul(c, ff{__ldg(a.ks + kvh), 0.f});
    c = ff_mul(c, ff{a.sm_hi, a.sm_lo});
    if (QG) {
      s_chi[row * (D / 32) + (lane >> 3)] = c.hi;   // per-slice scores are summed in fp32: the low part is not carried
    } else {
      s_chi[row] = c.hi;
      s_clo[row] = c.lo;
    }
  }
}

// 4 channels of row `row` of m tile `mt` for this lane (zeros for rows past the request's last query token).
template <int D, int NROWS>
__device__ __forceinline__ uint2 q_load_row(const DecodeArgs& a, int tok, int qlen, int kvh, int mt, int row, int lane) {
  const int R = mt * 16 + row, rt = R / a.G, rh = R - rt * a.G;
  uint2 raw = make_uint2(0u, 0u);
  if (row < NROWS && rt < qlen && lane < D / 4)
    raw = *reinterpret_cast<const uint2*>(a.q + (tok + rt) * a.q_st + (kvh * a.G + rh) * a.q_sh + lane * 4);
  return raw;
}
template <int D>
__device__ __forceinline__ void q_load_scale(const DecodeArgs& a, int kvh, int lane, float (&sk)[4]) {
  sk[0] = sk[1] = sk[2] = sk[3] = 1.f;   // a per-head K scale is not folded into q
  if (a.pc_k) {
    const float4 t4 = __ldg(reinterpret_cast<const float4*>(a.ks + kvh * D + (lane < D / 4 ? lane : 0) * 4));
    sk[0] = t4.x, sk[1] = t4.y, sk[2] = t4.z, sk[3] = t4.w;
  }
}

// q fold + quantize for the rows of m tile `mt` of (request, kv head): one warp per row in a rolled loop (this code
// runs once per item; kept small because straight-line code that is executed once mostly waits on instruction
// fetch). The next row's q is loaded while the current one is processed.
template <int D, int NROWS, bool QG = false>
__device__ __forceinline__ void q_prologue(const DecodeArgs& a, int8_t* s_q, float* s_chi, float* s_clo, int tok,
                                           int qlen, int kvh, int mt, int warp, int lane) {
  float sk[4];
  q_load_scale<D>(a, kvh, lane, sk);
  uint2 cur = q_load_row<D, NROWS>(a, tok, qlen, kvh, mt, warp, lane);
#pragma unroll 1
  for (int row = warp; row < NROWS; row += NWARPS) {
    const uint2 nxt = q_load_row<D, NROWS>(a, tok, qlen, kvh, mt, row + NWARPS, lane);
    q_quantize_row<D, QG>(a, cur, sk, s_q, s_chi, s_clo, kvh, row, lane);
    cur = nxt;
  }
}

// Four ints -> four int8 bytes (a lowest), each saturated to [-128, 127]: two saturating packs. cvt.pack puts its
// first source in bits 15:8, the second in bits 7:0 and the low half of the third operand in bits 31:16.
__device__ __forceinline__ uint32_t pack4_sat8(int a, int b, int c, int d) {
  uint32_t hi, r;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(d), "r"(c), "r"(0));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(b), "r"(a), "r"(hi));
  return r;
}

// Packed fp32 pairs (sm_100: add / mul / fma .f32x2 are two IEEE operations in one instruction).
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 pk2(float a, float b) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void upk2(f32x2 v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
// Scores of two dots of one row: fp32(dot * c) for c = hi + lo. The product is formed to ~48 bits and rounded once,
// like the reference's float(double(dot) * c). Plain fp32 would round c first and then the product; at |score| ~ 100
// that moves P = exp(score - max) by 1e-5 and flips its int8 quantization far more often than the reference's own
// noise. nhi = -hi (packed pair).
__device__ __forceinline__ f32x2 ints_to_f32x2(int d0, int d1) { return pk2(static_cast<float>(d0), static_cast<float>(d1)); }
__device__ __forceinline__ void score2(int d0, int d1, f32x2 hi, f32x2 nhi, f32x2 lo, float& s0, float& s1) {
  const f32x2 d = ints_to_f32x2(d0, d1);
  const f32x2 pn = mul2(d, nhi);                       // -(d * hi), rounded
  upk2(sub2(fma2(d, lo, fma2(d, hi, pn)), pn), s0, s1);   // p + (d * lo + (d * hi - p))
}

// Per-warp state of one m tile: q fragments, score scales, causal limits, running softmax statistics, output.
template <int D, bool ROWS16, bool QG = false>
struct TileState {
  uint32_t qa[D / 32][4];
  float ch0, cl0, ch1, cl1;            // one score scale per row (hi + lo)
  float cg0[QG ? D / 32 : 1], cg1[QG ? D / 32 : 1];   // QG: one score scale per (row, 32-channel slice)
  int lim0, lim1;
  float m0, m1, l0, l1;
  float acc[D / 8][ROWS16 ? 4 : 2];
};

// One 32-key chunk: S = Q.K^T, online softmax, P -> int8, O += P.V. sk / sv: shared-memory addresses of the
// swizzled K and V tiles; n_base: absolute position of the chunk's first key.
// The 16-row kernel (multi-token queries) is bound by its instruction stream (ncu: issue slots 56 %, DRAM 18 %), so its
// step is trimmed where the 8-row step is not (SLIM): mma accumulators start from the zero register instead of being
// cleared, causal masking is a branch only the last chunks of an item take, and the ldmatrix addresses come from three
// lane constants (~780 -> ~675 warp instructions per chunk and m tile, config 3 -7 %). The 8-row decode step keeps its
// instruction sequence on purpose: at large batches its loop runs at the rate HBM serves every SM fairly, and faster
// variants of it measured slower end to end.
template <int D, bool ROWS16, bool QG>
__device__ __forceinline__ void chunk_step(TileState<D, ROWS16, QG>& s, uint32_t sk, uint32_t sv, int n_base, int lim_all,
                                           int krow, int kmat, int vrow, int t, int hs, int hsel) {
  constexpr int KSTEPS = D / 32, NT = D / 8;
  constexpr bool SLIM = ROWS16;
  // 16-row tiles never run in head-group mode (hs = 1, hsel = 0). There the swizzle bits of a row depend on the lane
  // alone, tile_off(8 j + krow, c) = 8 j D + tile_off(krow, c) and tile_off(vrow, jp) = tile_off(vrow, 0) ^ (jp << 4):
  // two K bases and one V base per chunk, the rest are immediate offsets and one XOR per V load.
  const uint32_t ka0 = sk + tile_off<D>(krow, kmat), ka1 = sk + tile_off<D>(krow, (KSTEPS > 2 ? 4 : 0) + kmat);
  const uint32_t va = sv + tile_off<D>(vrow, 0);
  auto k_addr = [&](int j, int s2) {
    return SLIM ? (s2 ? ka1 : ka0) + j * 8 * D : sk + tile_off<D>(8 * j + krow, 4 * s2 + kmat, hs, hsel);
  };
  auto v_addr = [&](int jp) { return SLIM ? va ^ (jp << 4) : sv + tile_off<D>(vrow, jp, hs, hsel); };
  // accumulator (j, e) of lane (g, t): row g (e < 2) or g + 8, key n_base + 8j + 2t + (e & 1)
  const bool need_mask = n_base + CHUNK > lim_all;
  float p0[8], p1[8];
  float mx0 = -INFINITY, mx1 = -INFINITY;
  if constexpr (QG) {
    // S = Q.K^T with one q scale per 32-channel slice: every k step of the mma is one slice; its integer dot is scaled
    // by the slice's scale and the slices are summed in fp32
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      f32x2 a0 = pk2(0.f, 0.f), a1 = pk2(0.f, 0.f);
#pragma unroll
      for (int s2 = 0; s2 < KSTEPS / 2; ++s2) {
        uint32_t b[4];
        ldsm_x4(b, k_addr(j, s2));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          int d[4];
          d[0] = d[1] = d[2] = d[3] = 0;
          mma_s8(d, s.qa[2 * s2 + h], b[2 * h], b[2 * h + 1]);
          const float c0 = s.cg0[2 * s2 + h], c1 = s.cg1[2 * s2 + h];
          a0 = fma2(ints_to_f32x2(d[0], d[1]), pk2(c0, c0), a0);
          if (ROWS16) a1 = fma2(ints_to_f32x2(d[2], d[3]), pk2(c1, c1), a1);
        }
      }
      upk2(a0, p0[2 * j], p0[2 * j + 1]);
      if (ROWS16) upk2(a1, p1[2 * j], p1[2 * j + 1]);
    }
  }
  // S = Q.K^T: 4 n-tiles of 8 keys, natural key order
  int sacc[4][4];
  if constexpr (!QG) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (!SLIM) sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0;
#pragma unroll
      for (int s2 = 0; s2 < KSTEPS / 2; ++s2) {
        uint32_t b[4];
        ldsm_x4(b, k_addr(j, s2));
        if (SLIM && s2 == 0)
          mma_s8_zero(sacc[j], s.qa[0], b[0], b[1]);
        else
          mma_s8(sacc[j], s.qa[2 * s2], b[0], b[1]);
        mma_s8(sacc[j], s.qa[2 * s2 + 1], b[2], b[3]);
      }
    }
  }
  const f32x2 hi0 = pk2(s.ch0, s.ch0), nhi0 = pk2(-s.ch0, -s.ch0), lo0 = pk2(s.cl0, s.cl0);
  const f32x2 hi1 = pk2(s.ch1, s.ch1), nhi1 = pk2(-s.ch1, -s.ch1), lo1 = pk2(s.cl1, s.cl1);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if constexpr (!QG) {
      score2(sacc[j][0], sacc[j][1], hi0, nhi0, lo0, p0[2 * j], p0[2 * j + 1]);
      if (ROWS16) score2(sacc[j][2], sacc[j][3], hi1, nhi1, lo1, p1[2 * j], p1[2 * j + 1]);
    }
    if (!SLIM) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int n = n_base + 8 * j + 2 * t + e;
        if (need_mask && n >= s.lim0) p0[2 * j + e] = -INFINITY;
        mx0 = fmaxf(mx0, p0[2 * j + e]);
        if (ROWS16) {
          if (need_mask && n >= s.lim1) p1[2 * j + e] = -INFINITY;
          mx1 = fmaxf(mx1, p1[2 * j + e]);
        }
      }
    }
  }
  if (SLIM) {
    // only an item's last chunks reach a row's causal limit: the masking stays off the common path
    if (need_mask) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int n = n_base + 8 * (k >> 1) + 2 * t + (k & 1);
        if (n >= s.lim0) p0[k] = -INFINITY;
        if (ROWS16 && n >= s.lim1) p1[k] = -INFINITY;
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      mx0 = fmaxf(mx0, p0[k]);
      if (ROWS16) mx1 = fmaxf(mx1, p1[k]);
    }
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  const float mn0 = fmaxf(s.m0, mx0), nb0 = -mn0 * LOG2E;
  // m0 == mn0 also covers the "nothing seen yet" sentinel, where the fma below would see -1e30 * LOG2E cancel badly
  const float al0 = (s.m0 == mn0) ? 1.f : ex2(fmaf(s.m0, LOG2E, nb0));
  // the tile maximum of P is pexp(mx): the same instructions compute every P below, and they are monotonic
  const float ps0 = fmaxf(ex2(fmaf(mx0, LOG2E, nb0)) * (1.f / 127.f), 1e-30f);
  const float ri0 = __frcp_rn(ps0);
  // P = min(rint(exp2(.) / ps), 127) as int8: round to int, then saturating packs (cvt.pack.sat) build the A operand of
  // the PV mma directly (k slots 4t..4t+3 <- keys {2t, 2t+1, 8+2t, 9+2t}, slots 16+.. <- +16) and a byte dot product
  // with ones gives the row sum.
  const f32x2 l2e = pk2(LOG2E, LOG2E);
  auto quant8 = [&](const float (&p)[8], float nbx, float rix, uint32_t& lo4, uint32_t& hi4) {
    const f32x2 nb = pk2(nbx, nbx), ri = pk2(rix, rix);
    int q[8];
#pragma unroll
    for (int k = 0; k < 8; k += 2) {
      float x0, x1;
      upk2(fma2(pk2(p[k], p[k + 1]), l2e, nb), x0, x1);
      upk2(mul2(pk2(ex2(x0), ex2(x1)), ri), x0, x1);
      q[k] = __float2int_rn(x0), q[k + 1] = __float2int_rn(x1);
    }
    lo4 = pack4_sat8(q[0], q[1], q[2], q[3]);
    hi4 = pack4_sat8(q[4], q[5], q[6], q[7]);
    return __dp4a(static_cast<int>(lo4), 0x01010101, __dp4a(static_cast<int>(hi4), 0x01010101, 0));
  };
  uint32_t pa[4] = {0u, 0u, 0u, 0u};
  int qs0 = quant8(p0, nb0, ri0, pa[0], pa[2]);
  float al1 = 1.f, ps1 = 0.f;
  if (ROWS16) {
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn1 = fmaxf(s.m1, mx1), nb1 = -mn1 * LOG2E;
    al1 = (s.m1 == mn1) ? 1.f : ex2(fmaf(s.m1, LOG2E, nb1));
    ps1 = fmaxf(ex2(fmaf(mx1, LOG2E, nb1)) * (1.f / 127.f), 1e-30f);
    const int qs1 = quant8(p1, nb1, __frcp_rn(ps1), pa[1], pa[3]);
    s.m1 = mn1;
    qs0 |= qs1 << 16;  // both row sums (each < 2^13) through one pair of shuffles
  }
  s.m0 = mn0;
  qs0 += __shfl_xor_sync(0xffffffffu, qs0, 1);
  qs0 += __shfl_xor_sync(0xffffffffu, qs0, 2);
  if (ROWS16) {
    s.l1 = s.l1 * al1 + static_cast<float>(qs0 >> 16) * ps1;
    qs0 &= 0xffff;
  }
  s.l0 = s.l0 * al0 + static_cast<float>(qs0) * ps0;

  const f32x2 al0_2 = pk2(al0, al0), ps0_2 = pk2(ps0, ps0), al1_2 = pk2(al1, al1), ps1_2 = pk2(ps1, ps1);
  // O += P.V: 16 channels (two n-tiles) per transposing ldmatrix
#pragma unroll
  for (int jp = 0; jp < NT / 2; ++jp) {
    uint32_t b[4];
    ldsm_t8_x2(b, v_addr(jp));
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      int pacc[4];
      if (SLIM) {
        mma_s8_zero(pacc, pa, b[h2], b[2 + h2]);
      } else {
        pacc[0] = pacc[1] = pacc[2] = pacc[3] = 0;
        mma_s8(pacc, pa, b[h2], b[2 + h2]);
      }
      float* o = s.acc[2 * jp + h2];
      // (o0, o1) = (x0, x1) * ps + (o0, o1) * al
      upk2(fma2(ints_to_f32x2(pacc[0], pacc[1]), ps0_2, mul2(pk2(o[0], o[1]), al0_2)), o[0], o[1]);
      if (ROWS16)
        upk2(fma2(ints_to_f32x2(pacc[2], pacc[3]), ps1_2, mul2(pk2(o[2], o[3]), al1_2)), o[2], o[3]);
    }
  }
}

// QG: one q scale per 32 channels (kvq_int8_decode_attention_qgroup); otherwise one per row.
template <int D, bool ROWS16, bool QG>
__global__ void __launch_bounds__(NTHREADS, (Geom<D, ROWS16>::MIN_CTAS))
    decode_kernel(const DecodeArgs a, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
  using Gm = Geom<D, ROWS16>;
  constexpr int KSTEPS = D / 32, NT = D / 8, QROW = Gm::QROW, ACC_RS = Gm::ACC_RS, NSTG = Gm::NSTG, NSTAGE = Gm::NSTAGE;
  constexpr int NROWS = ROWS16 ? 16 : 8;
  // head groups exist only in single-token decode (the host never sets them for 16-row tiles): a constant there.
  // (A macro rather than a variable, so that the 8-row kernel keeps reading the launch parameter where it did.)
#define hgm (ROWS16 ? 0 : a.hg)
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_full[NSTG];    // TMA landed in the stage
  __shared__ __align__(8) uint64_t s_empty[NSTG];   // every warp of the group is done with the stage
  __shared__ int s_req, s_p0, s_f0, s_ubeg, s_uend;
  __shared__ unsigned long long s_scan[NWARPS];

  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
  int8_t* s_q = reinterpret_cast<int8_t*>(ring_ptr + Gm::RING);                       // [SLOTS][16][QROW]
  float* s_chi = reinterpret_cast<float*>(ring_ptr + Gm::RING + Gm::SLOTS * 16 * QROW);  // [64] score scale, high part
  float* s_clo = s_chi + 64;            // [64] score scale, low part
  float* s_m = s_clo + 64;              // [NWARPS][16] running max per warp
  float* s_l = s_m + 64;                // [NWARPS][16] denominator per warp
  float* s_M = s_l + 64;                // [slot][16] combined max
  float* s_inv = s_M + 64;              // [slot][16] 1 / combined denominator (whole item) or the denominator (cut item)
  float* s_acc = reinterpret_cast<float*>(ring_ptr);  // [NWARPS][NROWS][ACC_RS], valid between chunk loops

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  // Barriers start out partitioned for single-warp groups (decode); re-partitioned below if a request needs more.
  if (tid == 0) {
    for (int i = 0; i < NSTG; ++i) mbar_init(smem_u32(&s_full[i]), 1), mbar_init(smem_u32(&s_empty[i]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  fence_proxy_async();   // ordered before the first TMA issue by the __syncthreads of the request search below
  pdl_wait();            // everything above overlapped the plan kernel; its results are read from here on
  pdl_launch_dependents();
  // ---- this CTA's slice [ubeg, uend) of the global unit range (equal shares of the cost, see work_cost) and the
  //      request that owns its first unit ----
  const int P = a.item_cost;
  auto shape_of = [&](int r) {
    return req_shape(a.cu_q[r + 1] - a.cu_q[r], a.seq_lens[r], a.G, a.Hkv, a.qmax, a.grouped, hgm);
  };
  if (tid == 0) s_ubeg = 0x7fffffff, s_uend = -1;   // -1: the range ends with the last unit
  __syncthreads();
  int total, Wf;
  if (a.planned) {   // large batches: plan_kernel left the prefix sums of the per-request units and costs
    total = a.hdr[1], Wf = a.hdr[2];
    const int total_f = a.hdr[3], fb = blockIdx.x * Wf, fe = fb + Wf;
    const int32_t* prefix_f = a.prefix + a.num_seqs + 1;
    if (fb < total_f)
      for (int r = tid; r < a.num_seqs; r += NTHREADS) {
        const int f0r = prefix_f[r], f1r = prefix_f[r + 1];
        if (f0r <= fb && fb < f1r) s_req = r, s_p0 = a.prefix[r], s_f0 = f0r, s_ubeg = a.prefix[r] + unit_at_cost(shape_of(r), P, fb - f0r);
        if (f0r <= fe && fe < f1r) s_uend = a.prefix[r] + unit_at_cost(shape_of(r), P, fe - f0r);
      }
  } else {
    // every CTA sums units and costs itself: thread t takes a contiguous run of requests, the runs are scanned over the
    // block, and the threads whose runs contain the two ends of the CTA's cost range walk them again
    const int per = (a.num_seqs + NTHREADS - 1) / NTHREADS;
    const int r0 = tid * per, r1 = min(a.num_seqs, r0 + per);
    unsigned long long local = 0;   // cost in the high word, units in the low word
    for (int r = r0; r < r1; ++r) {
      const ReqShape rs = shape_of(r);
      local += (static_cast<unsigned long long>(work_cost(rs, P)) << 32) | static_cast<unsigned>(rs.units);
    }
    unsigned long long x = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) s_scan[warp] = x;
    __syncthreads();
    unsigned long long woff = 0, sum = 0;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) {
      if (w < warp) woff += s_scan[w];
      sum += s_scan[w];
    }
    total = static_cast<int>(sum & 0xffffffffu);
    const int total_f = static_cast<int>(sum >> 32);
    Wf = max((total_f + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x), MIN_UNITS);
    if (blockIdx.x == 0 && tid == 0) a.hdr[1] = total, a.hdr[2] = Wf, a.hdr[3] = total_f;
    const unsigned long long excl = woff + x - local;
    const int fb = blockIdx.x * Wf, fe = fb + Wf, ex_f = static_cast<int>(excl >> 32), lf = static_cast<int>(local >> 32);
    const bool has_b = ex_f <= fb && fb < ex_f + lf, has_e = ex_f <= fe && fe < ex_f + lf;
    if (has_b || has_e) {
      int p = static_cast<int>(excl & 0xffffffffu), f = ex_f;
      for (int r = r0; r < r1; ++r) {
        const ReqShape rs = shape_of(r);
        const int fr = work_cost(rs, P);
        if (has_b && f <= fb && fb < f + fr) s_req = r, s_p0 = p, s_f0 = f, s_ubeg = p + unit_at_cost(rs, P, fb - f);
        if (has_e && f <= fe && fe < f + fr) s_uend = p + unit_at_cost(rs, P, fe - f);
        p += rs.units, f += fr;
      }
    }
  }
  __syncthreads();
  const int ubeg = s_ubeg, uend = s_uend < 0 ? total : s_uend;
  // defaults: nothing is cut at the end of this CTA's range, no wait expired (overwritten below where that changes)
  if (tid == 0) a.bnd[blockIdx.x * 8] = -1, a.cta_status[blockIdx.x] = 0;
  if (ubeg >= uend) return;

  // Lane-constant pieces of the ldmatrix addresses.
  // K (non-transposed, 4 matrices of 8 keys x 16 channels): lane l addresses key (l & 7) of matrix l >> 3.
  // V (transposed 16x16 bytes): lane l addresses key vrow(l), chosen so that a lane's four bytes are the keys
  //   {2t, 2t+1, 8+2t, 9+2t} (+16 for the second matrix): the keys whose scores the same lane holds after QK.
  const int krow = lane & 7, kmat = lane >> 3;
  const int vrow = (lane & 1) + 8 * ((lane >> 1) & 1) + 2 * ((lane >> 2) & 3) + 16 * (lane >> 4);

  int cur_gs = 1;      // group size the barriers are currently initialised for
  int cst = 0, cpass = 0;  // consumer position of this warp's group in its ring: stage, completed passes
  bool ok = true;
  int u = ubeg;
  bool first_seg = true;
  int req = s_req, p0 = s_p0, f0 = s_f0;   // the request that owns unit u, its first unit and the cost before it;
                                           // later requests follow in order
  while (u < uend && req < a.num_seqs) {
    const int tok = a.cu_q[req], qlen = a.cu_q[req + 1] - tok, L = a.seq_lens[req];
    const ReqShape rs = req_shape(qlen, L, a.G, a.Hkv, a.qmax, a.grouped, hgm);
    if (rs.units == 0) {   // padding (q_len 0) and long requests have no work here
      ++req;
      continue;
    }
    const int nchunks = rs.nchunks;
    const int p1 = p0 + rs.units;
    const int32_t* bt = a.block_table + static_cast<int64_t>(req) * a.bt_stride;

    // The per-request code is compiled twice for 16-row tiles: once with the group size as the constant 4 (56 or more
    // rows per kv head, the multi-token case that is bound by its instruction stream: ring geometry, turn taking and
    // barrier addresses fold; config 3 -3.6 %), once generic. The 8-row kernel has the generic copy only.
    if constexpr (ROWS16) {
      if (rs.gs == 4) {
        constexpr int GS_C = 4;
#include "kvq_decode_request.inl"
      } else {
        constexpr int GS_C = 0;
#include "kvq_decode_request.inl"
      }
    } else {
      constexpr int GS_C = 0;
#include "kvq_decode_request.inl"
    }
    ++req;
    p0 = p1;
    f0 += work_cost(rs, P);
  }
}

// ------------------------------------------------------------------------------------------------------
// merge of items that were cut across CTAs
#undef hgm
// ------------------------------------------------------------------------------------------------------
constexpr int MERGE_THREADS = 256;
constexpr int MERGE_ROWS = 2;      // rows of an m tile per block: grid.y = 16 / MERGE_ROWS
constexpr int MERGE_SHALLOW = 8;   // up to this many partials per item: one lane group per row, no block cooperation

// One block per (CTA boundary, MERGE_ROWS rows of an m tile). Boundary b is where decode CTA b's range stops and CTA
// b + 1 starts; CTA b left a record saying which item (if any) it cut there as the first boundary inside the item,
// which of its two partial slots it used and the last CTA the item reaches, so an item cut by several boundaries is merged once and blocks of other boundaries exit after
// one load. The grid depends only on the decode grid, not on the batch. Two shapes of work:
//   shallow (the usual case, an item cut into a few partials): each group of D / 4 lanes owns one (m tile, row)
//     of the item and sums its partials itself, so the m tiles of a group merge side by side without a block barrier;
//   deep (one long request cut over hundreds of CTAs on an otherwise idle GPU): the partials of a row are spread
//     over the lane groups, MERGE_THREADS / (D / 4) in flight per step, and reduced through shared memory.
template <int D>
__global__ void __launch_bounds__(MERGE_THREADS) merge_kernel(const DecodeArgs a) {
  constexpr int LPP = D / 4, PG = MERGE_THREADS / LPP;   // lanes per partial row, lane groups per block
  static_assert(PG >= NWARPS * MERGE_ROWS, "a lane group per (m tile, row)");
  __shared__ float s_red[MERGE_THREADS / 32];
  __shared__ float4 s_num[PG][LPP];
  __shared__ float s_den[PG];
  pdl_wait();   // the records and partials below are written by the attention kernel
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x < 32) {
    // status word of the call: 1 if a bounded wait expired in any CTA of the attention kernel
    int bad = 0;
    for (int c = threadIdx.x; c <= static_cast<int>(gridDim.x); c += 32) bad |= a.cta_status[c];
    bad = __any_sync(0xffffffffu, bad != 0);
    if (threadIdx.x == 0) a.hdr[0] = bad;
  }
  const int4 r0 = *reinterpret_cast<const int4*>(a.bnd + blockIdx.x * 8);
  if (r0.x < 0) return;
  const int4 r1 = *reinterpret_cast<const int4*>(a.bnd + blockIdx.x * 8 + 4);
  const int kvh = r0.y, mg = r0.z, tok = r1.y, qlen = r1.z, gs = (r1.w >> 8) & 0xff, mtiles = r1.w & 0xff;
  const int tid = threadIdx.x;
  const int c_lo = blockIdx.x, c_hi = r1.x, lo_slot = (r1.w >> 16) & 1;
  const int lane = tid & 31, warp = tid >> 5, np = c_hi - c_lo + 1;
  const int pg = tid / LPP, l4 = tid - pg * LPP;
  // CTA c_lo reached this item after finishing earlier ones (second slot) unless its range starts with the item
  auto slot_of = [&](int c, int row) { return (c * 2 + (c == c_lo ? lo_slot : 0)) * a.part_rows + row; };
  // partial row = slot * 16 + row of the tile; slot = m tile of the group, or kv head of a head group
  auto store = [&](int sl, int r16, float4 t, float den) {
    const int mts = a.hg ? 0 : mg * gs + sl, kvs = kvh + (a.hg ? sl : 0);
    const int R = mts * 16 + r16, rt = R / a.G, rh = R - rt * a.G;
    const float inv = 1.f / fmaxf(den, 1e-30f);
    *reinterpret_cast<uint2*>(a.out + (tok + rt) * a.o_st + (kvs * a.G + rh) * a.o_sh + l4 * 4) =
        make_uint2(pack_bf16x2(t.x * inv, t.y * inv), pack_bf16x2(t.z * inv, t.w * inv));
  };
  auto live = [&](int sl, int r16) {
    const int mts = a.hg ? 0 : mg * gs + sl;
    return mts < mtiles && (mts * 16 + r16) / a.G < qlen;
  };

  if (np <= MERGE_SHALLOW) {
    const int sl = pg / MERGE_ROWS, r16 = blockIdx.y * MERGE_ROWS + (pg - sl * MERGE_ROWS);
    if (sl >= gs || !live(sl, r16)) return;
    const int row = sl * 16 + r16;
    float m[MERGE_SHALLOW], l[MERGE_SHALLOW];
    float4 x[MERGE_SHALLOW];
    float M = -1e30f;
#pragma unroll
    for (int i = 0; i < MERGE_SHALLOW; ++i)
      if (i < np) {   // every load of the row is issued before the first use
        const int ps = slot_of(c_lo + i, row);
        m[i] = a.part_ml[ps * 2];
        l[i] = a.part_ml[ps * 2 + 1];
        x[i] = *reinterpret_cast<const float4*>(a.part_acc + static_cast<int64_t>(ps) * D + l4 * 4);
      }
#pragma unroll
    for (int i = 0; i < MERGE_SHALLOW; ++i)
      if (i < np) M = fmaxf(M, m[i]);
    float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
    float den = 0.f;
#pragma unroll
    for (int i = 0; i < MERGE_SHALLOW; ++i)
      if (i < np) {
        const float w = ex2((m[i] - M) * LOG2E);
        num.x += w * x[i].x, num.y += w * x[i].y, num.z += w * x[i].z, num.w += w * x[i].w;
        den += w * l[i];
      }
    store(sl, r16, num, den);
    return;
  }

  for (int rb = 0; rb < MERGE_ROWS; ++rb)
    for (int sl = 0; sl < gs; ++sl) {   // uniform over the block
      const int r16 = blockIdx.y * MERGE_ROWS + rb, row = sl * 16 + r16;
      if (!live(sl, r16)) continue;
      float M = -1e30f;
      for (int i = tid; i < np; i += MERGE_THREADS) M = fmaxf(M, a.part_ml[slot_of(c_lo + i, row) * 2]);
#pragma unroll
      for (int o = 16; o; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
      if (lane == 0) s_red[warp] = M;
      __syncthreads();
#pragma unroll
      for (int w = 0; w < MERGE_THREADS / 32; ++w) M = fmaxf(M, s_red[w]);

      float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
      float den = 0.f;
#pragma unroll 4
      for (int i = pg; i < np; i += PG) {
        const int ps = slot_of(c_lo + i, row);
        const float w = ex2((a.part_ml[ps * 2] - M) * LOG2E);
        const float4 x = *reinterpret_cast<const float4*>(a.part_acc + static_cast<int64_t>(ps) * D + l4 * 4);
        num.x += w * x.x, num.y += w * x.y, num.z += w * x.z, num.w += w * x.w;
        den += w * a.part_ml[ps * 2 + 1];
      }
      s_num[pg][l4] = num;
      if (l4 == 0) s_den[pg] = den;
      __syncthreads();
      if (tid < LPP) {
        float4 t = s_num[0][tid];
        float dsum = s_den[0];
#pragma unroll
        for (int g = 1; g < PG; ++g) {   // fixed order: the result does not depend on scheduling
          const float4 x = s_num[g][tid];
          t.x += x.x, t.y += x.y, t.z += x.z, t.w += x.w;
          dsum += s_den[g];
        }
        store(sl, r16, t, dsum);
      }
      __syncthreads();   // s_red / s_num are reused by the next row
    }
}

// ------------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct DeviceInfo {
  bool ready = false;
  int sms = 0;
  int occ[2][2] = {{0, 0}, {0, 0}};  // [D == 128][ROWS16] resident CTAs per SM (the same with and without QG)
};

std::mutex g_mu;
DeviceInfo g_dev[64];
EncodeFn g_encode = nullptr;

struct MapKey {
  const void* ptr;
  int64_t nb, sb, sn, sh;
  int bs, H, D, box_heads;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && nb == o.nb && sb == o.sb && sn == o.sn && sh == o.sh && bs == o.bs && H == o.H && D == o.D &&
           box_heads == o.box_heads;
  }
};
struct MapEntry {
  MapKey key;
  CUtensorMap map;
  int pos[3];
};
std::vector<MapEntry> g_maps;

template <int D, bool R16>
int prepare_variant(int& occ) {
  KVQ_CUDA(cudaFuncSetAttribute(decode_kernel<D, R16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Geom<D, R16>::SMEM));
  KVQ_CUDA(cudaFuncSetAttribute(decode_kernel<D, R16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Geom<D, R16>::SMEM));
  int occ_qg = 0;
  KVQ_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, decode_kernel<D, R16, false>, NTHREADS, Geom<D, R16>::SMEM));
  KVQ_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ_qg, decode_kernel<D, R16, true>, NTHREADS, Geom<D, R16>::SMEM));
  occ = std::min(occ, occ_qg);
  occ = std::max(1, std::min(occ, MAX_CTAS_PER_SM));
  return KVQ_OK;
}

int device_info(DeviceInfo** out) {
  int dev = 0;
  KVQ_CUDA(cudaGetDevice(&dev));
  KVQ_REQUIRE(dev >= 0 && dev < 64, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceInfo& di = g_dev[dev];
  if (!di.ready) {
    KVQ_CUDA(cudaDeviceGetAttribute(&di.sms, cudaDevAttrMultiProcessorCount, dev));
    int rc;
    if ((rc = prepare_variant<64, false>(di.occ[0][0])) != KVQ_OK) return rc;
    if ((rc = prepare_variant<64, true>(di.occ[0][1])) != KVQ_OK) return rc;
    if ((rc = prepare_variant<128, false>(di.occ[1][0])) != KVQ_OK) return rc;
    if ((rc = prepare_variant<128, true>(di.occ[1][1])) != KVQ_OK) return rc;
    if (!g_encode) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      KVQ_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
      if (qres != cudaDriverEntryPointSuccess || !fn) {
        set_error("cuTensorMapEncodeTiled is not available from this driver");
        return KVQ_ERR_CUDA;
      }
      g_encode = reinterpret_cast<EncodeFn>(fn);
    }
    di.ready = true;
  }
  *out = &di;
  return KVQ_OK;
}

// Tensor map over a cache view [nb, bs, H, D] (int8). TMA wants ascending-friendly dims; the three outer dims are
// ordered by stride and pos[] tells the kernel which coordinate slot holds (slot-in-block, head, block).
// box_heads > 1 (head-group mode) needs adjacent heads (sh == D): the box is then [16 slots][box_heads][D] in smem.
int cache_tensor_map(const void* ptr, int64_t nb, int bs, int H, int D, int64_t sb, int64_t sn, int64_t sh,
                     int box_heads, CUtensorMap* map, int* pos) {
  const MapKey key{ptr, nb, sb, sn, sh, bs, H, D, box_heads};
  std::lock_guard<std::mutex> lock(g_mu);
  for (const MapEntry& e : g_maps)
    if (e.key == key) {
      *map = e.map;
      pos[0] = e.pos[0], pos[1] = e.pos[1], pos[2] = e.pos[2];
      return KVQ_OK;
    }
  struct Dim {
    int which;  // 0 slot-in-block, 1 head, 2 block
    uint64_t size, stride;
    uint32_t box;
  } dims[3] = {{0, static_cast<uint64_t>(bs), static_cast<uint64_t>(sn), 16u},
               {1, static_cast<uint64_t>(H), static_cast<uint64_t>(sh), static_cast<uint32_t>(box_heads)},
               {2, static_cast<uint64_t>(nb), static_cast<uint64_t>(sb), 1u}};
  for (Dim& d : dims)
    if (d.size == 1) d.stride = static_cast<uint64_t>(D);  // the stride of a size-1 dim is never used
  for (int i = 0; i < 3; ++i)
    for (int j = i + 1; j < 3; ++j)
      if (dims[j].stride < dims[i].stride) std::swap(dims[i], dims[j]);
  cuuint64_t gdim[4] = {static_cast<cuuint64_t>(D), dims[0].size, dims[1].size, dims[2].size};
  cuuint64_t gstr[3] = {dims[0].stride, dims[1].stride, dims[2].stride};
  cuuint32_t box[4] = {static_cast<cuuint32_t>(D), dims[0].box, dims[1].box, dims[2].box};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  MapEntry e;
  e.key = key;
  const CUresult r = g_encode(&e.map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(ptr), gdim, gstr, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, D == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                              box_heads > 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B
                                            : (D == 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_64B),
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (cache strides %lld/%lld/%lld)", static_cast<int>(r),
              static_cast<long long>(sb), static_cast<long long>(sn), static_cast<long long>(sh));
    return KVQ_ERR_CUDA;
  }
  for (int i = 0; i < 3; ++i) e.pos[dims[i].which] = i + 1;
  if (g_maps.size() >= 256) g_maps.clear();
  g_maps.push_back(e);
  *map = e.map;
  pos[0] = e.pos[0], pos[1] = e.pos[1], pos[2] = e.pos[2];
  return KVQ_OK;
}

// Launch with programmatic stream serialization: the kernel may begin while the previous kernel on the stream is
// still running and synchronises itself with pdl_wait().
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

cudaEvent_t g_ev_start = nullptr, g_ev_stop = nullptr;  // optional profiling brackets around decode_kernel

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct WorkspaceLayout {
  size_t prefix, bnd, status, part_acc, part_ml, total;
};
WorkspaceLayout workspace_layout(int num_seqs, int D, int max_ctas, int part_rows) {
  WorkspaceLayout w;
  w.prefix = HDR_BYTES;
  w.bnd = w.prefix + align_up(static_cast<size_t>(num_seqs + 1) * 8, 256);   // units and costs
  w.status = w.bnd + align_up(static_cast<size_t>(max_ctas) * 32, 256);
  w.part_acc = w.status + align_up(static_cast<size_t>(max_ctas) * 4, 256);
  w.part_ml = w.part_acc + static_cast<size_t>(max_ctas) * 2 * part_rows * D * 4;
  w.total = w.part_ml + static_cast<size_t>(max_ctas) * 2 * part_rows * 2 * 4;
  return w;
}

}  // namespace

int shared_device_sms(int* sms) {
  DeviceInfo* di = nullptr;
  const int rc = device_info(&di);
  if (rc == KVQ_OK) *sms = di->sms;
  return rc;
}
int shared_cache_tensor_map(const void* ptr, int64_t nb, int bs, int H, int D, int64_t sb, int64_t sn, int64_t sh,
                            int box_heads, CUtensorMap* map, int* pos) {
  return cache_tensor_map(ptr, nb, bs, H, D, sb, sn, sh, box_heads, map, pos);
}

}  // namespace kvq

using namespace kvq;

extern "C" __attribute__((visibility("default"))) size_t kvq_decode_workspace_size(int num_seqs, int head_dim) {
  DeviceInfo* di = nullptr;
  if (num_seqs < 0 || (head_dim != 64 && head_dim != 128) || device_info(&di) != KVQ_OK) return 0;
  // sized for the grouped mode (multi-token queries); single-token decode needs a quarter of the partial area
  return workspace_layout(num_seqs, head_dim, di->sms * MAX_CTAS_PER_SM, PART_ROWS_GROUPED).total;
}

extern "C" __attribute__((visibility("default"))) int kvq_decode_status(const void* workspace, int* status, kvq_stream_t stream) {
  KVQ_REQUIRE(workspace && status, "decode_status: null pointer");
  auto s = reinterpret_cast<cudaStream_t>(stream);
  KVQ_CUDA(cudaMemcpyAsync(status, workspace, sizeof(int), cudaMemcpyDeviceToHost, s));
  KVQ_CUDA(cudaStreamSynchronize(s));
  return KVQ_OK;
}

// What an item start costs a CTA, in units of its own work (one unit = one 32-key chunk of an item). The drained ring,
// the combination, the epilogue and the q prologue are ~5 us against ~0.35 us per unit in single-token decode (four
// streams per CTA), i.e. ~14 units; cutting an item also adds its partial rows and a merge. Measured over batch shapes
// (1 ... 128 requests x 32768, 128 x 4096, 256 x 1024, config 3): 14 ... 28 are equally good within 1-2 %, larger values
// lose (idle CTAs, uneven ranges); pairs of heads carry twice the bytes per unit.
static int item_cost_units(bool rows16, int hg) {
  static const int forced = [] {
    const char* e = getenv("KVQ_DECODE_ITEM_COST");   // tuning knob: overrides the built-in figures
    return e ? atoi(e) : -1;
  }();
  if (forced >= 0) return forced;
  (void)rows16;
  return hg ? 10 : 20;
}

// q_group: channels per q scale. 0 or head_dim: one scale per (query token, q head) row, the reference kernel's numerics;
// 32: one per 32-channel slice (the reference's q_gran="group32").
static int decode_attention_impl(const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* cu_q,
                                 const int32_t* seq_lens, const int32_t* block_table, const float* k_scale,
                                 const float* v_scale, double softmax_scale, int num_seqs, int num_q_heads, int num_kv_heads,
                                 int head_dim, int block_size, int64_t num_blocks, int64_t q_stride_t, int64_t q_stride_h,
                                 int64_t o_stride_t, int64_t o_stride_h, int64_t kc_stride_b, int64_t kc_stride_n,
                                 int64_t kc_stride_h, int64_t vc_stride_b, int64_t vc_stride_n, int64_t vc_stride_h,
                                 int64_t bt_stride, int k_per_channel, int v_per_channel, int max_query_len, int qmax,
                                 int q_group, void* workspace, size_t workspace_bytes, kvq_stream_t stream) {
  KVQ_REQUIRE(q_group == 0 || q_group == head_dim || q_group == 32, "q_group must be 0, head_dim or 32, got %d", q_group);
  KVQ_REQUIRE(head_dim == 64 || head_dim == 128, "head_dim must be 64 or 128, got %d", head_dim);
  KVQ_REQUIRE(block_size >= 16 && (block_size & (block_size - 1)) == 0, "block_size must be a power of two >= 16");
  KVQ_REQUIRE(num_kv_heads > 0 && num_q_heads > 0 && num_q_heads % num_kv_heads == 0, "bad head counts %d/%d",
              num_q_heads, num_kv_heads);
  KVQ_REQUIRE(qmax >= 1 && qmax <= 8, "qmax must be in [1, 8], got %d", qmax);
  KVQ_REQUIRE(num_seqs >= 0 && num_blocks > 0, "bad sizes");
  if (num_seqs == 0) return KVQ_OK;
  KVQ_REQUIRE(q && k_cache && v_cache && out && cu_q && seq_lens && block_table && k_scale && v_scale, "null pointer");
  KVQ_REQUIRE(aligned16(q) && aligned16(out) && q_stride_t % 8 == 0 && q_stride_h % 8 == 0 && o_stride_t % 8 == 0 &&
                  o_stride_h % 8 == 0,
              "q/out rows must be 16-byte aligned");
  KVQ_REQUIRE(aligned16(k_cache) && aligned16(v_cache) && kc_stride_b % 16 == 0 && kc_stride_n % 16 == 0 &&
                  kc_stride_h % 16 == 0 && vc_stride_b % 16 == 0 && vc_stride_n % 16 == 0 && vc_stride_h % 16 == 0,
              "cache rows must be 16-byte aligned");
  KVQ_REQUIRE(aligned16(k_scale) && aligned16(v_scale), "scales must be 16-byte aligned");
  DeviceInfo* di = nullptr;
  int rc = device_info(&di);
  if (rc != KVQ_OK) return rc;

  const int G = num_q_heads / num_kv_heads;
  const int max_q = std::max(1, std::min(max_query_len, qmax));
  const bool rows16 = G * max_q > 8;
  const int occ = di->occ[head_dim == 128][rows16];
  const int grid = di->sms * occ;
  // Multi-token queries with more than one m tile per kv head share K/V streams between warps (grouped mode); its
  // partial area is four times larger, so a workspace that only fits the plain layout falls back to one m tile
  // per item (same results, K/V re-read per m tile).
  const int mtiles_max = (G * max_q + 15) / 16;
  WorkspaceLayout wl = workspace_layout(num_seqs, head_dim, grid, PART_ROWS_GROUPED);
  int grouped = rows16 && mtiles_max >= 2 && workspace_bytes >= wl.total;
  // Head groups: single-tile decode over a token-major cache whose heads are adjacent in memory. With 8 or more
  // kv heads a (page, head) tile is 16 rows of head_dim bytes at a pitch of >= 1 KB, which HBM serves at ~75 % of
  // its rate; one stream per pair of adjacent heads reads 2 x head_dim contiguous bytes per key instead (measured
  // at Hkv = 8: 4.9 -> 5.9 TB/s with pairs, 5.1 TB/s with groups of four, which leave too few streams per SM;
  // at Hkv = 4 the plain mode is already at the HBM rate).
  int hg = 0;
  if (!rows16 && workspace_bytes >= wl.total && kc_stride_h == head_dim && vc_stride_h == head_dim &&
      kc_stride_n >= static_cast<int64_t>(num_kv_heads) * head_dim &&
      vc_stride_n >= static_cast<int64_t>(num_kv_heads) * head_dim && num_kv_heads >= 8 && num_kv_heads % 2 == 0)
    hg = 2;
  if (hg) grouped = 1;
  if (!grouped) wl = workspace_layout(num_seqs, head_dim, grid, PART_ROWS);
  if (!workspace || workspace_bytes < wl.total || (reinterpret_cast<uintptr_t>(workspace) & 255)) {
    set_error("decode workspace: need %zu bytes aligned to 256, got %zu at %p", wl.total, workspace_bytes, workspace);
    return KVQ_ERR_WORKSPACE;
  }

  DecodeArgs a;
  a.q = static_cast<const __nv_bfloat16*>(q), a.out = static_cast<__nv_bfloat16*>(out);
  a.cu_q = cu_q, a.seq_lens = seq_lens, a.block_table = block_table, a.ks = k_scale, a.vs = v_scale;
  auto* ws = static_cast<uint8_t*>(workspace);
  a.hdr = reinterpret_cast<int32_t*>(ws);
  a.prefix = reinterpret_cast<const int32_t*>(ws + wl.prefix);
  a.bnd = reinterpret_cast<int32_t*>(ws + wl.bnd);
  a.cta_status = reinterpret_cast<int32_t*>(ws + wl.status);
  a.planned = num_seqs > FUSED_PLAN_MAX;
  a.part_acc = reinterpret_cast<float*>(ws + wl.part_acc);
  a.part_ml = reinterpret_cast<float*>(ws + wl.part_ml);
  a.sm_hi = static_cast<float>(softmax_scale);
  a.sm_lo = static_cast<float>(softmax_scale - static_cast<double>(a.sm_hi));
  a.num_seqs = num_seqs, a.Hq = num_q_heads, a.Hkv = num_kv_heads, a.G = G, a.qmax = qmax;
  a.lbs = 0;
  while ((1 << a.lbs) < block_size) ++a.lbs;
  a.bs_mask = block_size - 1;
  a.q_st = q_stride_t, a.q_sh = q_stride_h, a.o_st = o_stride_t, a.o_sh = o_stride_h, a.bt_stride = bt_stride;
  a.pc_k = k_per_channel, a.pc_v = v_per_channel;
  a.grouped = grouped, a.hg = hg, a.part_rows = grouped ? PART_ROWS_GROUPED : PART_ROWS;
  a.item_cost = item_cost_units(rows16, hg);
  CUtensorMap tm_k, tm_v;
  if ((rc = cache_tensor_map(k_cache, num_blocks, block_size, num_kv_heads, head_dim, kc_stride_b, kc_stride_n,
                             kc_stride_h, hg ? hg : 1, &tm_k, a.kpos)) != KVQ_OK)
    return rc;
  if ((rc = cache_tensor_map(v_cache, num_blocks, block_size, num_kv_heads, head_dim, vc_stride_b, vc_stride_n,
                             vc_stride_h, hg ? hg : 1, &tm_v, a.vpos)) != KVQ_OK)
    return rc;

  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (a.planned)
    plan_kernel<<<1, 256, 0, s>>>(cu_q, seq_lens, num_seqs, G, num_kv_heads, qmax, grouped, hg, a.item_cost, grid, a.hdr,
                                  reinterpret_cast<int32_t*>(ws + wl.prefix));
  if (g_ev_start) KVQ_CUDA(cudaEventRecord(g_ev_start, s));
  const bool qg = q_group == 32;
  const dim3 mgrid(std::max(grid - 1, 1), 16 / MERGE_ROWS);
#define KVQ_LAUNCH_DECODE(DD, R16, QGG) \
  KVQ_CUDA(launch_pdl(decode_kernel<DD, R16, QGG>, dim3(grid), dim3(NTHREADS), Geom<DD, R16>::SMEM, s, a, tm_k, tm_v))
  if (head_dim == 128) {
    if (rows16) {
      if (qg) KVQ_LAUNCH_DECODE(128, true, true); else KVQ_LAUNCH_DECODE(128, true, false);
    } else {
      if (qg) KVQ_LAUNCH_DECODE(128, false, true); else KVQ_LAUNCH_DECODE(128, false, false);
    }
    if (g_ev_stop) KVQ_CUDA(cudaEventRecord(g_ev_stop, s));
    KVQ_CUDA(launch_pdl(merge_kernel<128>, mgrid, dim3(MERGE_THREADS), 0, s, a));
  } else {
    if (rows16) {
      if (qg) KVQ_LAUNCH_DECODE(64, true, true); else KVQ_LAUNCH_DECODE(64, true, false);
    } else {
      if (qg) KVQ_LAUNCH_DECODE(64, false, true); else KVQ_LAUNCH_DECODE(64, false, false);
    }
    if (g_ev_stop) KVQ_CUDA(cudaEventRecord(g_ev_stop, s));
    KVQ_CUDA(launch_pdl(merge_kernel<64>, mgrid, dim3(MERGE_THREADS), 0, s, a));
  }
#undef KVQ_LAUNCH_DECODE
  KVQ_CUDA(cudaGetLastError());
  return KVQ_OK;
}

extern "C" __attribute__((visibility("default"))) int kvq_int8_decode_attention(
    const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* cu_q, const int32_t* seq_lens,
    const int32_t* block_table, const float* k_scale, const float* v_scale, double softmax_scale, int num_seqs,
    int num_q_heads, int num_kv_heads, int head_dim, int block_size, int64_t num_blocks, int64_t q_stride_t,
    int64_t q_stride_h, int64_t o_stride_t, int64_t o_stride_h, int64_t kc_stride_b, int64_t kc_stride_n,
    int64_t kc_stride_h, int64_t vc_stride_b, int64_t vc_stride_n, int64_t vc_stride_h, int64_t bt_stride,
    int k_per_channel, int v_per_channel, int max_query_len, int qmax, void* workspace, size_t workspace_bytes,
    kvq_stream_t stream) {
  return decode_attention_impl(q, k_cache, v_cache, out, cu_q, seq_lens, block_table, k_scale, v_scale, softmax_scale,
                               num_seqs, num_q_heads, num_kv_heads, head_dim, block_size, num_blocks, q_stride_t, q_stride_h,
                               o_stride_t, o_stride_h, kc_stride_b, kc_stride_n, kc_stride_h, vc_stride_b, vc_stride_n,
                               vc_stride_h, bt_stride, k_per_channel, v_per_channel, max_query_len, qmax, 0, workspace,
                               workspace_bytes, stream);
}

extern "C" __attribute__((visibility("default"))) int kvq_int8_decode_attention_qgroup(
    const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* cu_q, const int32_t* seq_lens,
    const int32_t* block_table, const float* k_scale, const float* v_scale, double softmax_scale, int num_seqs,
    int num_q_heads, int num_kv_heads, int head_dim, int block_size, int64_t num_blocks, int64_t q_stride_t,
    int64_t q_stride_h, int64_t o_stride_t, int64_t o_stride_h, int64_t kc_stride_b, int64_t kc_stride_n,
    int64_t kc_stride_h, int64_t vc_stride_b, int64_t vc_stride_n, int64_t vc_stride_h, int64_t bt_stride,
    int k_per_channel, int v_per_channel, int max_query_len, int qmax, int q_group, void* workspace, size_t workspace_bytes,
    kvq_stream_t stream) {
  return decode_attention_impl(q, k_cache, v_cache, out, cu_q, seq_lens, block_table, k_scale, v_scale, softmax_scale,
                               num_seqs, num_q_heads, num_kv_heads, head_dim, block_size, num_blocks, q_stride_t, q_stride_h,
                               o_stride_t, o_stride_h, kc_stride_b, kc_stride_n, kc_stride_h, vc_stride_b, vc_stride_n,
                               vc_stride_h, bt_stride, k_per_channel, v_per_channel, max_query_len, qmax, q_group, workspace,
                               workspace_bytes, stream);
}

extern "C" __attribute__((visibility("default"))) int kvq_debug_decode_split(const int32_t* q_lens, const int32_t* seq_lens,
                                                                            int num_seqs, int group_size, int num_kv_heads,
                                                                            int qmax, int grouped, int head_group,
                                                                            int item_cost, int num_ctas, int32_t* ubeg,
                                                                            int32_t* uend) {
  // Host restatement of the split decode_kernel computes for itself (same req_shape / work_cost / unit_at_cost).
  KVQ_REQUIRE(q_lens && seq_lens && ubeg && uend && num_seqs >= 0 && num_ctas > 0 && group_size > 0 && num_kv_heads > 0,
              "decode_split: bad argument");
  if (item_cost < 0) item_cost = item_cost_units(group_size * std::min(std::max(qmax, 1), 8) > 8, head_group);
  std::vector<ReqShape> shapes(num_seqs);
  long long total = 0, total_f = 0;
  for (int r = 0; r < num_seqs; ++r) {
    shapes[r] = req_shape(q_lens[r], seq_lens[r], group_size, num_kv_heads, qmax, grouped, head_group);
    total += shapes[r].units, total_f += work_cost(shapes[r], item_cost);
  }
  KVQ_REQUIRE(total_f < (1ll << 31), "decode_split: more than 2^31 units");
  const int wf = std::max(static_cast<int>((total_f + num_ctas - 1) / num_ctas), MIN_UNITS);
  auto unit_of = [&](long long f) -> int {   // global unit at cost f
    if (f >= total_f) return static_cast<int>(total);
    long long p = 0, c = 0;
    for (int r = 0; r < num_seqs; ++r) {
      const int fr = work_cost(shapes[r], item_cost);
      if (f < c + fr) return static_cast<int>(p) + unit_at_cost(shapes[r], item_cost, static_cast<int>(f - c));
      p += shapes[r].units, c += fr;
    }
    return static_cast<int>(total);
  };
  for (int b = 0; b < num_ctas; ++b) {
    ubeg[b] = unit_of(static_cast<long long>(b) * wf);
    uend[b] = unit_of(static_cast<long long>(b + 1) * wf);
  }
  return KVQ_OK;
}

extern "C" __attribute__((visibility("default"))) int kvq_debug_kernel_events(void* start_event, void* stop_event) {
  g_ev_start = static_cast<cudaEvent_t>(start_event);
  g_ev_stop = static_cast<cudaEvent_t>(stop_event);
  return KVQ_OK;
}

// ------------------------------------------------------------------------------------------------------
// Attention without a caller-provided workspace.
//
// Some callers may not allocate device memory at all: a serving engine that has already handed every free
// byte to its KV-cache pool, a plugin running inside another framework's memory pool or while that framework
// captures a CUDA graph, a real-time loop where cudaMalloc's implicit synchronization is unacceptable. For
// them the scratch of the attention kernels (work plan, split-KV partials, status word) lives in a fixed
// array in the library's own device image. Every GPU that loads the library holds these KVQ_STATIC_WS_BYTES
// until the process exits.
// ------------------------------------------------------------------------------------------------------
namespace kvq {
namespace {

constexpr size_t KVQ_STATIC_WS_BYTES = 10u << 20;  // 10 MiB: enough for 592 CTAs (148 SMs x 4) and ~150k requests
static __device__ __align__(256) unsigned char g_static_ws[KVQ_STATIC_WS_BYTES];

// Device address of g_static_ws per device. In host code the symbol g_static_ws is only a stand-in: it must go
// through cudaGetSymbolAddress (with the device current) before a kernel can use it.
void* g_static_ws_ptr[64] = {};

int static_workspace(void** out) {
  int dev = 0;
  KVQ_CUDA(cudaGetDevice(&dev));
  KVQ_REQUIRE(dev >= 0 && dev < 64, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_static_ws_ptr[dev]) {
    void* p = nullptr;
    KVQ_CUDA(cudaGetSymbolAddress(&p, g_static_ws));
    g_static_ws_ptr[dev] = p;
  }
  *out = g_static_ws_ptr[dev];
  return KVQ_OK;
}

}  // namespace
}  // namespace kvq

extern "C" __attribute__((visibility("default"))) size_t kvq_static_workspace_bytes(void) { return KVQ_STATIC_WS_BYTES; }

extern "C" __attribute__((visibility("default"))) int kvq_int8_decode_attention_noalloc(
    const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* cu_q, const int32_t* seq_lens,
    const int32_t* block_table, const float* k_scale, const float* v_scale, double softmax_scale, int num_seqs,
    int num_q_heads, int num_kv_heads, int head_dim, int block_size, int64_t num_blocks, int64_t q_stride_t,
    int64_t q_stride_h, int64_t o_stride_t, int64_t o_stride_h, int64_t kc_stride_b, int64_t kc_stride_n,
    int64_t kc_stride_h, int64_t vc_stride_b, int64_t vc_stride_n, int64_t vc_stride_h, int64_t bt_stride,
    int k_per_channel, int v_per_channel, int max_query_len, int qmax, kvq_stream_t stream) {
  if (num_seqs > 0 && (head_dim == 64 || head_dim == 128)) {
    // the plain layout (one m tile per item) is enough: with it the call never needs more than this
    DeviceInfo* di = nullptr;
    const int rc0 = device_info(&di);
    if (rc0 != KVQ_OK) return rc0;
    const size_t need = workspace_layout(num_seqs, head_dim, di->sms * MAX_CTAS_PER_SM, PART_ROWS).total;
    if (need > KVQ_STATIC_WS_BYTES) {
      set_error("kvq_int8_decode_attention_noalloc: %d requests need %zu bytes of scratch, the built-in array holds %zu; "
                "use kvq_int8_decode_attention with a caller-provided workspace",
                num_seqs, need, static_cast<size_t>(KVQ_STATIC_WS_BYTES));
      return KVQ_ERR_WORKSPACE;
    }
  }
  void* ws = nullptr;
  const int rc = static_workspace(&ws);
  if (rc != KVQ_OK) return rc;
  return kvq_int8_decode_attention(q, k_cache, v_cache, out, cu_q, seq_lens, block_table, k_scale, v_scale, softmax_scale,
                                   num_seqs, num_q_heads, num_kv_heads, head_dim, block_size, num_blocks, q_stride_t,
                                   q_stride_h, o_stride_t, o_stride_h, kc_stride_b, kc_stride_n, kc_stride_h, vc_stride_b,
                                   vc_stride_n, vc_stride_h, bt_stride, k_per_channel, v_per_channel, max_query_len, qmax,
                                   ws, KVQ_STATIC_WS_BYTES, stream);
}

