// Causal flash attention for sm_100a (head dimension 128, bf16, GQA), forward and backward.
//
// Inputs live in one packed projection buffer [B, S, Hp, 128] with Hp = Hkv * (rep + 2) heads in
// group-major order (per KV head: its `rep` query heads, then the key head, then the value head),
// so query, key and value tiles are all fetched with the same 4-D TMA tensor map. Every matrix
// product runs on the tensor cores through tcgen05.mma with fp32 accumulators in TMEM:
//
//   forward  (128 query rows per CTA, 64 keys per step, two CTAs per SM so that one CTA's softmax
//             overlaps the other's MMAs):
//        S = Q K^T  -> TMEM (double buffered);  softmax threads (one per query row) read S,
//        keep a running maximum that is only raised when it grows by more than 2^8 (the
//        accumulator is then rescaled in TMEM), write P (bf16) to swizzled shared memory;
//        O += P V accumulates in TMEM; epilogue divides by the row sum.
//   backward (128 keys per CTA, 64 query rows per step, every query head of the KV group):
//        S^T = K Q^T, dP^T = V dO^T -> TMEM; threads (one per key row) form P^T and dS^T in
//        shared memory; dV += P^T dO, dK += dS^T Q accumulate in TMEM over the whole loop;
//        dQ^T = K^T dS^T is read back each step and added to an fp32 dQ buffer with
//        coalesced atomics (red.global.add.f32).
//
// Warp roles (both kernels): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, the
// others = softmax / epilogue (TMEM lane quarter = warp % 4; four warps forward, eight - two per
// quarter, splitting the columns - backward). The backward TMA warp also brings the step's
// log-sum-exp and delta rows into shared memory with the step's Q / dO tiles, two steps ahead of
// their use: as global loads of the compute warps they queued in the load/store unit behind the
// 32 dQ reductions every thread issues per step. All waits are bounded.
//
// Measured on the backward call (B4 H32 S2048, one GPU, alternating runs; 0.816 ms before): a
// three-stage Q / dO ring 0.793 ms, ex2.approx instead of exp2f 0.780 ms, the staged rows on top
// of the ring 0.700 ms (all kept; forward 0.252 -> 0.233 ms with ex2.approx). The same staging
// with a two-stage ring was slower (0.940 ms: the rows arrived with the tiles, one step ahead,
// and the compute warps waited for them). Also not kept: sixteen compute warps of 16 columns
// (3 % slower before the staging, 0.6 % faster after it), dQ through shared memory and cp.reduce.async.bulk (0.92 ms; 0.86 ms against 0.70
// with a reducer warp of its own), dQ reductions
// interleaved with the next step's exponentials (0.86 ms). A cycle-stamped trace of one CTA
// before these changes: 5,200 cycles per 64-query step, the eight compute warps busy for 4,500
// of them (exponentials 1,280, dS 970, the dQ reductions 1,320), the MMA lane issuing its 32
// small (N = 64) instructions in 2,300.
#include <math.h>

#include "host_common.h"
#include "ptx.cuh"

namespace mm {

constexpr int FA_D = 128;
constexpr int FA_THREADS = 192;
constexpr int MM_ERR_ATTN_WAIT = 7;    // an attention kernel gave up waiting on one of its barriers
constexpr int MM_ERR_ATTN_ALIGN = 8;   // dynamic shared memory was not 1024-byte aligned

// 2^x on the special-function unit alone (ex2.approx.ftz: relative error 2^-22, -inf -> 0): the
// library exp2f adds range scaling around the same instruction, which matters in loops whose
// length is set by the instruction count of one warp (forward: 0.251 -> 0.235 ms on B4 H32 S2048).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ------------------------------------------------------------------ forward
constexpr int FA_BM = 128;
constexpr int FA_BN = 64;
constexpr int FA_SQ = 2 * FA_BM * 128;  // two 64-column halves of 128 rows x 128 B
constexpr int FA_SKV = 2 * FA_BN * 128; // per stage
constexpr int FA_SP = FA_BM * 128;
constexpr int FA_FWD_SMEM = FA_SQ + 4 * FA_SKV + FA_SP + 128;

struct FaFwdParams {
  __nv_bfloat16* out;  // [B, S, Hq, 128]
  float* lse;          // [B, Hq, S]
  int S, Hkv, rep;
  float scale_log2;    // softmax scale * log2(e)
};

__global__ void __launch_bounds__(FA_THREADS, 2)
    flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
                     FaFwdParams p, int* __restrict__ err) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) atomicCAS(err, 0, MM_ERR_ATTN_ALIGN);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + FA_SQ;
  uint8_t* sV = sK + 2 * FA_SKV;
  uint8_t* sP = sV + 2 * FA_SKV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + FA_SP);
  uint64_t* q_full = bars;          // [1]
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* k_empty = bars + 3;     // [2]
  uint64_t* v_full = bars + 5;      // [2]
  uint64_t* v_empty = bars + 7;     // [2]
  uint64_t* s_full = bars + 9;      // [2]
  uint64_t* s_free = bars + 11;     // [2]
  uint64_t* p_ready = bars + 13;    // [1]
  uint64_t* pv_done = bars + 14;    // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_blk = gridDim.x - 1 - blockIdx.x;  // longest rows first
  const int hq = blockIdx.y, b = blockIdx.z;
  const int g = hq / p.rep, r = hq - g * p.rep;
  const int hp_q = g * (p.rep + 2) + r, hp_k = g * (p.rep + 2) + p.rep, hp_v = hp_k + 1;
  const int nblk = 2 * q_blk + 2;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 4);
    }
    mbar_init(p_ready, 4);
    mbar_init(pv_done, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmKV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base;        // two 64-column score buffers
  const uint32_t tO = tmem_base + 128;  // 128-column output accumulator

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, FA_SQ);
      tma_load_4d(sQ, &tmQ, q_full, 0, hp_q, q_blk * FA_BM, b);
      tma_load_4d(sQ + FA_BM * 128, &tmQ, q_full, 64, hp_q, q_blk * FA_BM, b);
      bool ok = true;
      for (int j = 0; j < nblk && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1, err, MM_ERR_ATTN_WAIT)) { ok = false; break; }
        mbar_expect_tx(&k_full[st], FA_SKV);
        tma_load_4d(sK + st * FA_SKV, &tmKV, &k_full[st], 0, hp_k, j * FA_BN, b);
        tma_load_4d(sK + st * FA_SKV + FA_BN * 128, &tmKV, &k_full[st], 64, hp_k, j * FA_BN, b);
        if (!mbar_wait(&v_empty[st], ph ^ 1, err, MM_ERR_ATTN_WAIT)) { ok = false; break; }
        mbar_expect_tx(&v_full[st], FA_SKV);
        tma_load_4d(sV + st * FA_SKV, &tmKV, &v_full[st], 0, hp_v, j * FA_BN, b);
        tma_load_4d(sV + st * FA_SKV + FA_BN * 128, &tmKV, &v_full[st], 64, hp_v, j * FA_BN, b);
      }
      if (!ok)
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);  // let copies in flight land before exit
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(FA_BM, FA_BN, false, false);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(FA_BM, FA_D, false, true);
      const uint32_t q_base = smem_u32(sQ), p_base = smem_u32(sP);
      auto issue_s = [&](int j) {
        const int st = j & 1;
        const uint32_t k_base = smem_u32(sK + st * FA_SKV);
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t da = umma_desc_sw128(q_base + h * (FA_BM * 128) + kk * 32, 16, 1024);
            const uint64_t db = umma_desc_sw128(k_base + h * (FA_BN * 128) + kk * 32, 16, 1024);
            umma_bf16(tS + st * FA_BN, da, db, idesc_s, (h | kk) ? 1u : 0u);
          }
        umma_commit(&s_full[st]);
        umma_commit(&k_empty[st]);
      };
      bool ok = mbar_wait(q_full, 0, err, MM_ERR_ATTN_WAIT) && mbar_wait(&k_full[0], 0, err, MM_ERR_ATTN_WAIT);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; j < nblk && ok; ++j) {
        if (j + 1 < nblk) {
          const int n = j + 1;
          if (!mbar_wait(&k_full[n & 1], (n >> 1) & 1, err, MM_ERR_ATTN_WAIT) ||
              !mbar_wait(&s_free[n & 1], ((n >> 1) & 1) ^ 1, err, MM_ERR_ATTN_WAIT)) { ok = false; break; }
          tc_fence_after();
          issue_s(n);
        }
        if (!mbar_wait(&v_full[j & 1], (j >> 1) & 1, err, MM_ERR_ATTN_WAIT) ||
            !mbar_wait(p_ready, j & 1, err, MM_ERR_ATTN_WAIT)) { ok = false; break; }
        tc_fence_after();
        const uint32_t v_base = smem_u32(sV + (j & 1) * FA_SKV);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t da = umma_desc_sw128(p_base + kk * 32, 16, 1024);
          const uint64_t db = umma_desc_sw128(v_base + kk * 2048, FA_BN * 128, 1024);
          umma_bf16(tO, da, db, idesc_pv, (j | kk) ? 1u : 0u);
        }
        umma_commit(pv_done);
        umma_commit(&v_empty[j & 1]);
      }
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int rowg = q_blk * FA_BM + row;
    const uint32_t lane_bits = static_cast<uint32_t>(q * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk; ++j) {
      const int sb = j & 1;
      if (ok && !mbar_wait(&s_full[sb], (j >> 1) & 1, err, MM_ERR_ATTN_WAIT)) ok = false;
      tc_fence_after();
      uint32_t s0[32], s1[32];
      tmem_ld_32x32(tS + lane_bits + sb * FA_BN, s0);
      tmem_ld_32x32(tS + lane_bits + sb * FA_BN + 32, s1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[sb]);
      const bool diag = j >= 2 * q_blk;  // the last two key blocks cross the diagonal
      const int col0 = j * FA_BN;
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float a = __uint_as_float(s0[c]) * p.scale_log2;
        float bb = __uint_as_float(s1[c]) * p.scale_log2;
        if (diag) {
          if (col0 + c > rowg) a = -INFINITY;
          if (col0 + 32 + c > rowg) bb = -INFINITY;
        }
        s0[c] = __float_as_uint(a);
        s1[c] = __float_as_uint(bb);
        mx = fmaxf(mx, fmaxf(a, bb));
      }
      if (j > 0) {
        if (ok && !mbar_wait(pv_done, (j - 1) & 1, err, MM_ERR_ATTN_WAIT)) ok = false;
        tc_fence_after();
      }
      const float m_new = fmaxf(m_used, mx);
      const bool need = m_new > m_used + 8.f;  // raise the reference maximum only on large growth
      float alpha = 1.f;
      if (need) {
        alpha = fast_exp2(m_used - m_new);
        m_used = m_new;
      }
      if (j > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(tO + lane_bits + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32(tO + lane_bits + c * 32, o);
        }
        tmem_st_wait();
      }
      l *= alpha;
      float sum = 0.f;
      uint8_t* prow = sP + row * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = ch * 8 + i;
          const float sv = __uint_as_float(c < 32 ? s0[c] : s1[c - 32]);
          e[i] = fast_exp2(sv - m_used);
          sum += e[i];
        }
        uint4 v;
        v.x = pack_bf16(e[0], e[1]);
        v.y = pack_bf16(e[2], e[3]);
        v.z = pack_bf16(e[4], e[5]);
        v.w = pack_bf16(e[6], e[7]);
        *reinterpret_cast<uint4*>(prow + ((ch ^ (row & 7)) * 16)) = v;
      }
      l += sum;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    if (ok && !mbar_wait(pv_done, (nblk - 1) & 1, err, MM_ERR_ATTN_WAIT)) ok = false;
    tc_fence_after();
    const float inv = 1.f / l;
    __nv_bfloat16* orow = p.out + ((static_cast<int64_t>(b) * p.S + rowg) * (p.Hkv * p.rep) + hq) * FA_D;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t o[32];
      tmem_ld_32x32(tO + lane_bits + c * 32, o);
      tmem_ld_wait();
      if (ok) {
        uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 v;
          v.x = pack_bf16(__uint_as_float(o[i * 8 + 0]) * inv, __uint_as_float(o[i * 8 + 1]) * inv);
          v.y = pack_bf16(__uint_as_float(o[i * 8 + 2]) * inv, __uint_as_float(o[i * 8 + 3]) * inv);
          v.z = pack_bf16(__uint_as_float(o[i * 8 + 4]) * inv, __uint_as_float(o[i * 8 + 5]) * inv);
          v.w = pack_bf16(__uint_as_float(o[i * 8 + 6]) * inv, __uint_as_float(o[i * 8 + 7]) * inv);
          dst[i] = v;
        }
      }
    }
    if (ok) p.lse[(static_cast<int64_t>(b) * (p.Hkv * p.rep) + hq) * p.S + rowg] = m_used * 0.6931471805599453f + logf(l);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// ------------------------------------------------------------------ backward
constexpr int FB_BKV = 128;
constexpr int FB_BQ = 64;
constexpr int FB_SKV = 2 * FB_BKV * 128;  // K or V: 32 KiB
constexpr int FB_SQ = 2 * FB_BQ * 128;    // Q or dO stage: 16 KiB
constexpr int FB_SPT = FB_BKV * 128;      // P^T or dS^T: 16 KiB
// Stages of the Q / dO ring. The MMA lane waits for the tiles of step n + 1 before it turns to the
// products of step n, so with two stages every step also paid the latency of a TMA load that
// could only be issued when step n - 1 had released its stage (0.816 -> 0.793 ms on B4 H32 S2048).
constexpr int FB_QST = 3;
constexpr int FB_SROW = 2 * FB_BQ * 4;    // per stage: log-sum-exp and delta of the step's 64 query rows
constexpr int FB_SMEM = 2 * FB_SKV + 2 * FB_QST * FB_SQ + 2 * FB_SPT + 256 + FB_QST * FB_SROW;

struct FaBwdParams {
  const float* lse;    // [B, Hq, S]
  const float* delta;  // [B, Hq, S]  rowsum(dO * O)
  float* dq_acc;       // [B, S, Hq, 128] fp32, zero on entry
  __nv_bfloat16* dqkv; // packed [B, S, Hp, 128]
  int S, Hkv, rep;
  float scale, scale_log2;
};

constexpr int FB_THREADS = 320;   // TMA warp, MMA warp, eight compute warps
__global__ void __launch_bounds__(FB_THREADS, 1)
    flash_bwd_kernel(const __grid_constant__ CUtensorMap tmKV, const __grid_constant__ CUtensorMap tmQ,
                     const __grid_constant__ CUtensorMap tmDO, FaBwdParams p, int* __restrict__ err) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) atomicCAS(err, 0, MM_ERR_ATTN_ALIGN);
    return;
  }
  uint8_t* sK = smem;
  uint8_t* sV = sK + FB_SKV;
  uint8_t* sQ = sV + FB_SKV;              // [FB_QST stages]
  uint8_t* sDO = sQ + FB_QST * FB_SQ;     // [FB_QST stages]
  uint8_t* sPT = sDO + FB_QST * FB_SQ;
  uint8_t* sDST = sPT + FB_SPT;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDST + FB_SPT);
  uint64_t* kv_full = bars;                      // [1]
  uint64_t* qdo_full = bars + 1;                 // [FB_QST]
  uint64_t* qdo_empty = qdo_full + FB_QST;       // [FB_QST]
  uint64_t* st_full = qdo_empty + FB_QST;        // [2]
  uint64_t* st_free = st_full + 2;               // [2]
  uint64_t* dpt_full = st_free + 2;              // [1]
  uint64_t* dpt_free = dpt_full + 1;             // [1]
  uint64_t* ps_ready = dpt_free + 1;             // [1]
  uint64_t* dqt_full = ps_ready + 1;             // [1]
  uint64_t* dqt_free = dqt_full + 1;             // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dqt_free + 1);
  float* sRow = reinterpret_cast<float*>(sDST + FB_SPT + 256);   // [FB_QST][lse 64 | delta 64]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jb = blockIdx.x;  // key block; block 0 has the most query blocks and starts first
  const int g = blockIdx.y, b = blockIdx.z;
  const int Hq = p.Hkv * p.rep;
  const int hp_k = g * (p.rep + 2) + p.rep, hp_v = hp_k + 1;
  const int i0 = jb * (FB_BKV / FB_BQ);
  const int nq = p.S / FB_BQ - i0;      // query blocks at or below the diagonal
  const int nsteps = nq * p.rep;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < FB_QST; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&st_full[i], 1);
      mbar_init(&st_free[i], 8);
    }
    mbar_init(dpt_full, 1);
    mbar_init(dpt_free, 8);
    mbar_init(ps_ready, 8);
    mbar_init(dqt_full, 1);
    mbar_init(dqt_free, 8);
    fence_barrier_init();
    tma_prefetch_desc(&tmKV);
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmDO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tST = tmem_base;         // 2 x 64 columns
  const uint32_t tDPT = tmem_base + 128;  // 64
  const uint32_t tDQT = tmem_base + 192;  // 64
  const uint32_t tDV = tmem_base + 256;   // 128
  const uint32_t tDK = tmem_base + 384;   // 128

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * FB_SKV);
      tma_load_4d(sK, &tmKV, kv_full, 0, hp_k, jb * FB_BKV, b);
      tma_load_4d(sK + FB_BKV * 128, &tmKV, kv_full, 64, hp_k, jb * FB_BKV, b);
      tma_load_4d(sV, &tmKV, kv_full, 0, hp_v, jb * FB_BKV, b);
      tma_load_4d(sV + FB_BKV * 128, &tmKV, kv_full, 64, hp_v, jb * FB_BKV, b);
      bool ok = true;
      for (int n = 0; n < nsteps && ok; ++n) {
        const int st = n % FB_QST;
        const int r = n / nq, i = i0 + (n - r * nq);
        const int hq = g * p.rep + r, hp_q = g * (p.rep + 2) + r;
        if (!mbar_wait(&qdo_empty[st], ((n / FB_QST) & 1) ^ 1, err, MM_ERR_ATTN_WAIT)) { ok = false; break; }
        mbar_expect_tx(&qdo_full[st], 2 * FB_SQ + FB_SROW);
        {
          const int64_t row_off = (static_cast<int64_t>(b) * Hq + hq) * p.S + i * FB_BQ;
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                           smem_u32(sRow + st * (2 * FB_BQ))),
                       "l"(p.lse + row_off), "r"(FB_BQ * 4), "r"(smem_u32(&qdo_full[st]))
                       : "memory");
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                           smem_u32(sRow + st * (2 * FB_BQ) + FB_BQ)),
                       "l"(p.delta + row_off), "r"(FB_BQ * 4), "r"(smem_u32(&qdo_full[st]))
                       : "memory");
        }
        tma_load_4d(sQ + st * FB_SQ, &tmQ, &qdo_full[st], 0, hp_q, i * FB_BQ, b);
        tma_load_4d(sQ + st * FB_SQ + FB_BQ * 128, &tmQ, &qdo_full[st], 64, hp_q, i * FB_BQ, b);
        tma_load_4d(sDO + st * FB_SQ, &tmDO, &qdo_full[st], 0, hq, i * FB_BQ, b);
        tma_load_4d(sDO + st * FB_SQ + FB_BQ * 128, &tmDO, &qdo_full[st], 64, hq, i * FB_BQ, b);
      }
      if (!ok)
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_st = umma_idesc_bf16(FB_BKV, FB_BQ, false, false);   // K Q^T, V dO^T
      constexpr uint32_t idesc_acc = umma_idesc_bf16(FB_BKV, FA_D, false, true);    // P^T dO, dS^T Q
      constexpr uint32_t idesc_dqt = umma_idesc_bf16(FA_D, FB_BQ, true, true);      // K^T dS^T
      const uint32_t k_base = smem_u32(sK), v_base = smem_u32(sV);
      const uint32_t pt_base = smem_u32(sPT), dst_base = smem_u32(sDST);
      auto issue_scores = [&](uint32_t tdst, uint32_t a_base, uint32_t b_base) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t da = umma_desc_sw128(a_base + h * (FB_BKV * 128) + kk * 32, 16, 1024);
            const uint64_t db = umma_desc_sw128(b_base + h * (FB_BQ * 128) + kk * 32, 16, 1024);
            umma_bf16(tdst, da, db, idesc_st, (h | kk) ? 1u : 0u);
          }
      };
      bool ok = mbar_wait(kv_full, 0, err, MM_ERR_ATTN_WAIT) && mbar_wait(&qdo_full[0], 0, err, MM_ERR_ATTN_WAIT);
      if (ok) {
        tc_fence_after();
        issue_scores(tST, k_base, smem_u32(sQ));
        umma_commit(&st_full[0]);
        issue_scores(tDPT, v_base, smem_u32(sDO));
        umma_commit(dpt_full);
      }
      for (int n = 0; n < nsteps && ok; ++n) {
        const int st = n % FB_QST;
        if (n + 1 < nsteps) {
          const int m = n + 1, ms = m & 1, mq = m % FB_QST;
          if (!mbar_wait(&qdo_full[mq], (m / FB_QST) & 1, err, MM_ERR_ATTN_WAIT) ||
              !mbar_wait(&st_free[ms], ((m >> 1) & 1) ^ 1, err, MM_ERR_ATTN_WAIT)) { ok = false; break; }
          tc_fence_after();
          issue_scores(tST + ms * FB_BQ, k_base, smem_u32(sQ + mq * FB_SQ));
          umma_commit(&st_full[ms]);
          if (!mbar_wait(dpt_free, n & 1, err, MM_ERR_ATTN_WAIT)) { ok = false; break; }
          tc_fence_after();
          issue_scores(tDPT, v_base, smem_u32(sDO + mq * FB_SQ));
          umma_commit(dpt_full);
        }
        if (!mbar_wait(ps_ready, n & 1, err, MM_ERR_ATTN_WAIT)) { ok = false; break; }
        tc_fence_after();
        const uint32_t q_base = smem_u32(sQ + st * FB_SQ), do_base = smem_u32(sDO + st * FB_SQ);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {   // dV += P^T dO   (K = 64 query rows)
          const uint64_t da = umma_desc_sw128(pt_base + kk * 32, 16, 1024);
          const uint64_t db = umma_desc_sw128(do_base + kk * 2048, FB_BQ * 128, 1024);
          umma_bf16(tDV, da, db, idesc_acc, (n | kk) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {   // dK += dS^T Q
          const uint64_t da = umma_desc_sw128(dst_base + kk * 32, 16, 1024);
          const uint64_t db = umma_desc_sw128(q_base + kk * 2048, FB_BQ * 128, 1024);
          umma_bf16(tDK, da, db, idesc_acc, (n | kk) ? 1u : 0u);
        }
        if (!mbar_wait(dqt_free, (n & 1) ^ 1, err, MM_ERR_ATTN_WAIT)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {   // dQ^T = K^T dS^T   (K = 128 key rows)
          const uint64_t da = umma_desc_sw128(k_base + kk * 2048, FB_BKV * 128, 1024);
          const uint64_t db = umma_desc_sw128(dst_base + kk * 2048, FB_BKV * 128, 1024);
          umma_bf16(tDQT, da, db, idesc_dqt, kk ? 1u : 0u);
        }
        umma_commit(dqt_full);
        umma_commit(&qdo_empty[st]);
      }
    }
  } else {
    // Eight compute warps: two per TMEM lane quarter, each handling 32 of the step's 64 query
    // columns, so the serial chain per step (TMEM load, exp, products, shared-memory stores,
    // reductions) is half as long as with one warp per quarter.
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;      // 0: query columns 0..31 of the step, 1: columns 32..63
    const int t = q * 32 + lane;           // key row of this thread (also the d index for dQ^T)
    const int kvg = jb * FB_BKV + t;
    const uint32_t lane_bits = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t col_off = static_cast<uint32_t>(half * 32);
    const float log2e = 1.4426950408889634f;
    bool ok = true;
    uint32_t dq_regs[32];
    int prev_hq = 0, prev_i = 0;
    auto flush_dq = [&](int hq, int i) {
      // lane = d: 32 consecutive floats per warp and query row -> one 128-byte reduction
      float* base = p.dq_acc + ((static_cast<int64_t>(b) * p.S + i * FB_BQ + half * 32) * Hq + hq) * FA_D + t;
#pragma unroll
      for (int c = 0; c < 32; ++c) atomicAdd(base + static_cast<int64_t>(c) * Hq * FA_D, __uint_as_float(dq_regs[c]));
    };
    for (int n = 0; n < nsteps; ++n) {
      const int sb = n & 1;
      const int r = n / nq, i = i0 + (n - r * nq);
      const int hq = g * p.rep + r;
      const int qcol0 = i * FB_BQ + half * 32;   // first query row (global) of this warp's columns
      const float* lse_row = sRow + (n % FB_QST) * (2 * FB_BQ) + half * 32;
      const float* delta_row = lse_row + FB_BQ;
      const bool diag = i < i0 + FB_BKV / FB_BQ;
      // ---- P^T (st_full follows the MMA lane's wait for the stage's qdo_full, which also covers the rows)
      if (ok && !mbar_wait(&qdo_full[n % FB_QST], (n / FB_QST) & 1, err, MM_ERR_ATTN_WAIT)) ok = false;
      if (ok && !mbar_wait(&st_full[sb], (n >> 1) & 1, err, MM_ERR_ATTN_WAIT)) ok = false;
      tc_fence_after();
      uint32_t pk[16], dsk[16];
      {
        uint32_t s0[32];
        tmem_ld_32x32(tST + lane_bits + sb * FB_BQ + col_off, s0);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&st_free[sb]);
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const float4 ls = *(reinterpret_cast<const float4*>(lse_row) + c4);
          const float lv[4] = {ls.x, ls.y, ls.z, ls.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int c = c4 * 4 + u;
            float e = fast_exp2(__uint_as_float(s0[c]) * p.scale_log2 - lv[u] * log2e);
            if (diag && kvg > qcol0 + c) e = 0.f;
            s0[c] = __float_as_uint(e);
          }
        }
        // ---- dS^T
        if (ok && !mbar_wait(dpt_full, n & 1, err, MM_ERR_ATTN_WAIT)) ok = false;
        tc_fence_after();
        uint32_t d0[32];
        tmem_ld_32x32(tDPT + lane_bits + col_off, d0);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(dpt_free);
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const float4 dl = *(reinterpret_cast<const float4*>(delta_row) + c4);
          const float dv[4] = {dl.x, dl.y, dl.z, dl.w};
          float pe[4], de[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int c = c4 * 4 + u;
            pe[u] = __uint_as_float(s0[c]);
            de[u] = pe[u] * (__uint_as_float(d0[c]) - dv[u]) * p.scale;
          }
          pk[c4 * 2] = pack_bf16(pe[0], pe[1]);
          pk[c4 * 2 + 1] = pack_bf16(pe[2], pe[3]);
          dsk[c4 * 2] = pack_bf16(de[0], de[1]);
          dsk[c4 * 2 + 1] = pack_bf16(de[2], de[3]);
        }
      }
      // ---- dQ^T of the previous step; its completion also frees sPT / sDST
      if (n > 0) {
        if (ok && !mbar_wait(dqt_full, (n - 1) & 1, err, MM_ERR_ATTN_WAIT)) ok = false;
        tc_fence_after();
        tmem_ld_32x32(tDQT + lane_bits + col_off, dq_regs);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(dqt_free);
      }
      // ---- publish this warp's 32 columns (four 16-byte units per row) of P^T and dS^T
      uint8_t* prow = sPT + t * 128;
      uint8_t* drow = sDST + t * 128;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        const int phys = ((half * 4 + ch) ^ (t & 7)) * 16;
        *reinterpret_cast<uint4*>(prow + phys) = make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
        *reinterpret_cast<uint4*>(drow + phys) = make_uint4(dsk[ch * 4], dsk[ch * 4 + 1], dsk[ch * 4 + 2], dsk[ch * 4 + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ps_ready);
      if (n > 0 && ok) flush_dq(prev_hq, prev_i);
      prev_hq = hq;
      prev_i = i;
    }
    // last dQ^T, then the dK / dV accumulators
    if (ok && !mbar_wait(dqt_full, (nsteps - 1) & 1, err, MM_ERR_ATTN_WAIT)) ok = false;
    tc_fence_after();
    tmem_ld_32x32(tDQT + lane_bits + col_off, dq_regs);
    tmem_ld_wait();
    if (ok) flush_dq(prev_hq, prev_i);
    const int Hp = p.Hkv * (p.rep + 2);
    __nv_bfloat16* krow = p.dqkv + ((static_cast<int64_t>(b) * p.S + kvg) * Hp + hp_k) * FA_D;
    __nv_bfloat16* vrow = krow + FA_D;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      const uint32_t tsrc = which ? tDV : tDK;
      __nv_bfloat16* dst_row = which ? vrow : krow;
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {     // this warp's half of the 128 columns
        const int c = half * 2 + cc;
        uint32_t o[32];
        tmem_ld_32x32(tsrc + lane_bits + c * 32, o);
        tmem_ld_wait();
        if (ok) {
          uint4* dst = reinterpret_cast<uint4*>(dst_row + c * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(o[i * 8 + 0]), __uint_as_float(o[i * 8 + 1]));
            v.y = pack_bf16(__uint_as_float(o[i * 8 + 2]), __uint_as_float(o[i * 8 + 3]));
            v.z = pack_bf16(__uint_as_float(o[i * 8 + 4]), __uint_as_float(o[i * 8 + 5]));
            v.w = pack_bf16(__uint_as_float(o[i * 8 + 6]), __uint_as_float(o[i * 8 + 7]));
            dst[i] = v;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]; half a warp per row with 16-byte loads,
// four rows per warp so that four loads per lane are in flight.
__global__ void flash_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                                   float* __restrict__ delta, int B, int S, int Hq) {
  const int64_t warp_id = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int half = lane >> 4, l16 = lane & 15;
  const int64_t total = static_cast<int64_t>(B) * S * Hq;
  const int64_t r[2] = {warp_id * 4 + half, warp_id * 4 + 2 + half};   // rows are (b, s, h)
  uint4 a[2], c[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int64_t rk = r[k] < total ? r[k] : 0;
    a[k] = *reinterpret_cast<const uint4*>(dout + rk * FA_D + l16 * 8);
    c[k] = *reinterpret_cast<const uint4*>(out + rk * FA_D + l16 * 8);
  }
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const uint32_t aw[4] = {a[k].x, a[k].y, a[k].z, a[k].w}, cw[4] = {c[k].x, c[k].y, c[k].z, c[k].w};
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = unpack_bf16(aw[j]), y = unpack_bf16(cw[j]);
      s += x.x * y.x + x.y * y.y;
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (l16 == 0 && r[k] < total) {
      const int h = static_cast<int>(r[k] % Hq);
      const int64_t bs = r[k] / Hq;
      const int sidx = static_cast<int>(bs % S);
      const int64_t bidx = bs / S;
      delta[(bidx * Hq + h) * S + sidx] = s;
    }
  }
}

// dq_acc fp32 [B, S, Hq, 128] -> bf16 query slots of the packed gradient buffer.
__global__ void flash_dq_store_kernel(const float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dqkv, int64_t rows,
                                      int Hkv, int rep) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;  // one thread per 8 values
  if (idx >= rows * (FA_D / 8)) return;
  const int64_t row = idx / (FA_D / 8);   // (b, s, hq)
  const int part = static_cast<int>(idx % (FA_D / 8));
  const int Hq = Hkv * rep;
  const int hq = static_cast<int>(row % Hq);
  const int64_t bs = row / Hq;
  const int g = hq / rep, r = hq - g * rep;
  const float4 x = *reinterpret_cast<const float4*>(dq_acc + row * FA_D + part * 8);
  const float4 y = *reinterpret_cast<const float4*>(dq_acc + row * FA_D + part * 8 + 4);
  uint4 v;
  v.x = pack_bf16(x.x, x.y);
  v.y = pack_bf16(x.z, x.w);
  v.z = pack_bf16(y.x, y.y);
  v.w = pack_bf16(y.z, y.w);
  const int64_t Hp = static_cast<int64_t>(Hkv) * (rep + 2);
  *reinterpret_cast<uint4*>(dqkv + (bs * Hp + g * (rep + 2) + r) * FA_D + part * 8) = v;
}

static int packed_map(CUtensorMap* out, const void* base, int B, int S, int H, int box_rows) {
  const uint64_t dims[4] = {static_cast<uint64_t>(FA_D), static_cast<uint64_t>(H), static_cast<uint64_t>(S),
                            static_cast<uint64_t>(B)};
  const uint64_t strides[4] = {0, static_cast<uint64_t>(FA_D) * 2, static_cast<uint64_t>(H) * FA_D * 2,
                               static_cast<uint64_t>(S) * H * FA_D * 2};
  const uint32_t box[4] = {64, 1, static_cast<uint32_t>(box_rows), 1};
  return encode_tmap_bf16(out, base, 4, dims, strides, box, 1);
}

}  // namespace mm

extern "C" {

// 1 when (S, D) can run on the tcgen05 attention kernels.
int mm_flash_attn_supported(int S, int D) { return (D == mm::FA_D && S >= 128 && S % 128 == 0) ? 1 : 0; }

// qkv: packed bf16 [B, S, Hkv*(rep+2), 128] (contiguous); out: bf16 [B, S, Hkv*rep, 128];
// lse: fp32 [B, Hkv*rep, S]. Causal, scale 1/sqrt(128).
int mm_flash_attn_fwd(const void* qkv, void* out, float* lse, int B, int S, int Hkv, int rep, int D,
                      cudaStream_t stream) {
  using namespace mm;
  if (!mm_flash_attn_supported(S, D)) return -2;
  DeviceState* ds = device_state();
  if (!ds) return -1;
  const int Hp = Hkv * (rep + 2);
  CUtensorMap tmQ, tmKV;
  int rc = packed_map(&tmQ, qkv, B, S, Hp, FA_BM);
  if (rc) return rc;
  rc = packed_map(&tmKV, qkv, B, S, Hp, FA_BN);
  if (rc) return rc;
  static bool configured[kMaxDevices] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev]) {
    MM_CUDA_TRY(cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_FWD_SMEM));
    configured[dev] = true;
  }
  FaFwdParams p;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.S = S;
  p.Hkv = Hkv;
  p.rep = rep;
  p.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(D));
  dim3 grid(S / FA_BM, Hkv * rep, B);
  flash_fwd_kernel<<<grid, FA_THREADS, FA_FWD_SMEM, stream>>>(tmQ, tmKV, p, ds->status);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

// dqkv: packed bf16 gradient buffer, same layout as qkv (every element is written).
// dq_acc: fp32 scratch [B, S, Hkv*rep, 128]; delta: fp32 scratch [B, Hkv*rep, S].
int mm_flash_attn_bwd(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv,
                      float* dq_acc, float* delta, int B, int S, int Hkv, int rep, int D, cudaStream_t stream) {
  using namespace mm;
  if (!mm_flash_attn_supported(S, D)) return -2;
  DeviceState* ds = device_state();
  if (!ds) return -1;
  const int Hp = Hkv * (rep + 2), Hq = Hkv * rep;
  CUtensorMap tmKV, tmQ, tmDO;
  int rc = packed_map(&tmKV, qkv, B, S, Hp, FB_BKV);
  if (rc) return rc;
  rc = packed_map(&tmQ, qkv, B, S, Hp, FB_BQ);
  if (rc) return rc;
  rc = packed_map(&tmDO, dout, B, S, Hq, FB_BQ);
  if (rc) return rc;
  static bool configured[kMaxDevices] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev]) {
    MM_CUDA_TRY(cudaFuncSetAttribute(flash_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FB_SMEM));
    configured[dev] = true;
  }
  const int64_t rows = static_cast<int64_t>(B) * S * Hq;
  MM_CUDA_TRY(cudaMemsetAsync(dq_acc, 0, rows * FA_D * sizeof(float), stream));
  {
    const int threads = 256;
    const int64_t blocks = ((rows + 3) / 4 * 32 + threads - 1) / threads;
    flash_delta_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(out), delta, B, S, Hq);
  }
  FaBwdParams p;
  p.lse = lse;
  p.delta = delta;
  p.dq_acc = dq_acc;
  p.dqkv = static_cast<__nv_bfloat16*>(dqkv);
  p.S = S;
  p.Hkv = Hkv;
  p.rep = rep;
  p.scale = 1.f / sqrtf(static_cast<float>(D));
  p.scale_log2 = p.scale * 1.4426950408889634f;
  dim3 grid(S / FB_BKV, Hkv, B);
  flash_bwd_kernel<<<grid, FB_THREADS, FB_SMEM, stream>>>(tmKV, tmQ, tmDO, p, ds->status);
  {
    const int threads = 256;
    const int64_t n = rows * (FA_D / 8);
    flash_dq_store_kernel<<<static_cast<unsigned>((n + threads - 1) / threads), threads, 0, stream>>>(
        dq_acc, static_cast<__nv_bfloat16*>(dqkv), rows, Hkv, rep);
  }
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

}  // extern "C"
