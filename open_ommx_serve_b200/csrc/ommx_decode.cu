// Paged decode attention over OMMX-quantized KV planes for sm_100a: split-KV stage 1, stage 2
// (log-sum-exp combine with the bf16 sink/recent rows fused in) and the partial-state merge.
//
// Stage 1 replaces _canonical_splitkv_stage1 (ommx_gpu_serve/attention/paged_decode.py:1255-2284
// of the reference).  One CTA serves one (split, sequence) pair and ALL local kv heads of its
// token range, so every page row it touches is a full contiguous line:
//
//   producer warp   streams whole pages / group-slot planes into a shared-memory ring: the two
//                   code planes through swizzled tensor maps, the small planes with 1-D bulk
//                   copies, completion through mbarrier transaction counts; page ids, group
//                   slots and the copy roles of a stage are tabulated in shared memory once.
//   15 decode warps build, two per (group, kv head) unit, the unit's sidecar tile: outlier
//                   deltas (bit walk with clz, FP4 nibble, base code byte) as fp16
//                   [token][channel], the fp32 q.zp dot products of the unit's query heads, and the
//                   power-of-two K and V scale factors laid out in MMA-fragment order.
//   8 MMA warps     own one unit per stage and a private online-softmax state.  All MMAs are
//                   m16n8k16 fp16 with the 2-bit codes as the A operand - a code field masked in
//                   place is the fp16 subnormal code * 4^slot * 2^-24, exact and offset-free - and
//                   the query heads as the 8 columns: logits = codes.(q*2^e) + delta.q + (q.zp from the sidecar),
//                   softmax over token rows, P transposed with movmatrix, output =
//                   codes^T.(P*2^e_v) + vz^T.P.
//
// Numerics follow the reference kernel's rounding points: q*sm_scale rounded to bf16, exact
// code*2^e products, the outlier delta rounded to bf16, q.zp as an fp32 dot product of the raw
// query with the zero-points (paged_decode.py:1754-1770), fp32 accumulation, V as exact code*2^e
// products with the zero-point bias summed apart.  One point differs inside the gate: P is rounded
// to fp16 (11 bits) instead of bf16.
#include "ommx_common.cuh"
#include <cuda.h>                       // CUtensorMap (types only; the encoder is looked up at run time)
#include <mutex>
#include <stdlib.h>
#include <string.h>

namespace ommx {

constexpr int HD = 128;                 // head_dim this build serves
constexpr int NCW = 8;                  // (group, head) units in flight per CTA, one MMA warp each
// Two warp layouts.  Narrow (4 or 8 local kv heads: 14 copies per ring stage): 15 decode warps + 1 producer warp, which
// also builds the last tile half once its copies are out.  Wide (1 or 2 local kv heads: a stage is 8 or 4 groups, 112 or
// 56 small copies): 16 decode warps + 4 producer warps, because one warp issues a bulk copy only every ~60 cycles and
// the issues of different warps overlap (112 copies: 6400 cycles from one warp, 2000 from four).
template <bool WIDE> struct WarpLayout {
    static constexpr int NDW = WIDE ? 16 : 15;            // decode warps (stateless sidecar builders, items dealt round-robin)
    static constexpr int NPW = WIDE ? 4 : 1;              // producer warps
    static constexpr int PRODUCER_WARP = NCW + NDW;       // the first of them
    static constexpr int THREADS = (NCW + NDW + NPW) * 32;
};
// Register budget per role (setmaxnreg, warpgroup granularity).  Only what the CTA was launched with
// can be moved around: 768 threads x 80 = 61440 = 256*128 (MMA) + 512*56 (decode + producer).  The
// launch refuses to run if the compiled kernel holds fewer registers than the roles ask for, because
// setmaxnreg.inc would then wait forever.
#define OMMX_REGS_MMA "128"
#define OMMX_REGS_DECODE "56"
#define OMMX_REGS_PRODUCER "24"
constexpr int REGS_MMA = 128, REGS_DECODE = 56, REGS_PRODUCER = 24;
constexpr int MAX_STAGES = 4;           // ring depth (3 when the planes of a stage are large)
constexpr int DT_STRIDE = 272;          // bytes per sidecar-tile row (256 data + 16 pad)
constexpr int ROW_ZP = 32;              // q.zp partial sums, fp32: [channel half][8 query heads of the kv head]
constexpr int ROW_KF = 33;              // K scale factors 2^(e+4), fp16, in code-fragment order
constexpr int ROW_VF = 34;              // V scale factors, fp16, fragment order (rows 34, 35: two copies)
constexpr int ROW_ZT = 36;              // V zero-points [scale group][token], fp16 (rows 36, 37: two copies)
constexpr int DT_ROWS = 38;             // rows 0..31: outlier deltas [token][channel], fp16
constexpr int DT_BYTES = DT_ROWS * DT_STRIDE;
constexpr int MAX_SPLIT_GROUPS = 512;   // groups one CTA can index (16K tokens per split)
constexpr int MAX_SPLIT_PAGES = 1024;
constexpr long long WAIT_LIMIT_CYCLES = 2000000000ll;   // about a second of SM clock: the wait has failed

struct S1Params {
    const __nv_bfloat16 *q;
    int64_t q_sb, q_sh;
    int32_t B, Hq, H, gqa, q_vec_ok;     // q_vec_ok: eight adjacent q elements may be fetched as one 16-byte word
    const uint8_t *k_base, *v_main, *v_scale, *v_zp, *k_scale, *k_zp, *k_ms, *k_mc, *k_obmp, *k_oval;
    int32_t ps, ppg, num_pages, num_slots, k_out, nb, use_map;
    int32_t nbi;                         // bytes of outlier index per channel: 4 (flat bitmask) or ceil(7k/8) (relidx7, idx7 = 1)
    int32_t idx7;
    const int32_t *b_seq_len;
    const void *r2t, *r2g;
    int32_t tbl64;
    int64_t r2t_sb, r2g_sb;
    float *al;
    int64_t al_sb, al_sh, al_ss;
    int32_t S, seg_group_base;
    float sm_scale, logit_cap;
    int32_t *status;
    int32_t abl;
    // shared-memory layout of one group block (bytes)
    int32_t GS, gb_bytes, stage_bytes, nstages, hshift;
    int32_t o_vm, o_vs, o_vz, o_ks, o_kz, o_ms, o_mc, o_bm, o_ov;
    // tensor maps of the two code planes as [bytes/128][128] uint8 with 128-byte swizzle
    uint32_t swz;                        // 0x70 when the maps are in use, else 0
    int32_t rows_per_page;               // 128-byte lines per page
    alignas(64) CUtensorMap tmap_k;
    alignas(64) CUtensorMap tmap_v;
};

// One bulk copy of a stage: source plane, bytes, destination inside the stage, and which table entry
// (page id or group slot) selects the source block.
struct __align__(16) CopyDesc {
    const uint8_t *src;                  // plane base, or nullptr + kind for a tensor-map copy
    uint32_t unit, dst;
    int32_t tbase, tmul, gi, tok0;       // gi: group in stage (bits 0..7) | kind << 8
};                                       // kind 0 bulk copy, 1 k_base through tmap_k, 2 v_main through tmap_v
// a stage holds at most 8 groups x (4 planes x 4 pages + 6 group planes) = 176 copies (1 kv head, 8-token pages)

// ---- PTX wrappers --------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: returns false (and the caller raises OMMX_ST_TIMEOUT) instead of spinning forever.
// try_wait already parks the warp in hardware for a short while.  The limit is counted on the SM
// clock (cheap to read); nanosleep or the global timer in this loop would put their own latency
// on every producer/consumer hand-off.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, long long limit = WAIT_LIMIT_CYCLES) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const long long t_end = clock64() + limit;
#pragma unroll 1
    for (uint32_t i = 1;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 0 && clock64() > t_end) return false;
    }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x2(uint32_t addr, uint32_t &r0, uint32_t &r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
// transpose an 8x8 matrix of 16-bit elements held one row pair per lane (the accumulator layout)
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(x));
    return r;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t hmul2_f16(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The 2-bit code planes are staged with the TMA's 128-byte swizzle (16-byte chunk index XOR line
// index mod 8) when a page is a whole number of 1 KB swizzle atoms: a head's 32-byte code row then
// lands in a different bank window on each token row instead of the same one.  `o` is the linear byte
// offset inside a 1 KB aligned region; swz is 0x70 (swizzled) or 0 (plain bulk copies).
__device__ __forceinline__ uint32_t swz128(uint32_t o, uint32_t swz) { return o ^ ((o >> 3) & swz); }

__device__ __forceinline__ void tma_2d_g2s(uint32_t dst, const CUtensorMap *map, int32_t x, int32_t y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

__device__ __forceinline__ int64_t load_index(const void *tbl, int is64, int64_t i) {
    return is64 ? reinterpret_cast<const int64_t *>(tbl)[i] : (int64_t) reinterpret_cast<const int32_t *>(tbl)[i];
}

// =================================================================================================
// Stage 1
// =================================================================================================
// Ablation bits (differential timing only, they break parity; mirror of the reference's
// OMMX_ABL_* knobs, paged_decode.py:3267-3279): 1 = skip the outlier splice, 2 = skip V dequant
// and P.V, 4 = skip the K code dequant and its MMAs.
constexpr int ABL_NO_OUTLIER = 1, ABL_NO_V = 2, ABL_NO_K = 4, ABL_NO_COMPUTE = 8;   // 8: stream the planes only
// 16 (tests of the give-up path only): waits give up after about 2 ms and the producer announces the bytes of its
// second ring fill without issuing the copies, so that every role runs out of patience and leaves through the epilogue
constexpr int ABL_TEST_STALL = 16;
constexpr long long TEST_WAIT_LIMIT_CYCLES = 4000000ll;

// fp16 bits of 2^(e + FBIAS).  Exponents below -18 give 0 (such a scale step is under 2^-18 and the
// term it multiplies is dropped); exponents above 11 are clamped and reported.
constexpr int FBIAS = 4;
__device__ __forceinline__ uint32_t pow2_f16_bits(int e, bool &clamped) {
    int u = e + 15 + FBIAS;
    clamped = u > 30;
    u = min(u, 30);
    return u < 1 ? 0u : (uint32_t)u << 10;
}
// the reference rounds an outlier's delta to bf16; keep that rounding point, then store it as fp16
// (exact: 8 significant bits fit in 11)
__device__ __forceinline__ uint32_t f16_bits_of_bf16_rounded(float x) {
    uint16_t r;
    const float xb = bf16_round_f32(x);
    asm("cvt.rn.satfinite.f16.f32 %0, %1;" : "=h"(r) : "f"(xb));
    return (uint32_t)r;
}
__device__ __forceinline__ uint32_t f16_bits_sat(float x) {
    uint16_t r;
    asm("cvt.rn.satfinite.f16.f32 %0, %1;" : "=h"(r) : "f"(x));
    return (uint32_t)r;
}
// field i (0..7) of the lower and upper 8 codes of a 32-bit code word, as two fp16 subnormals
// code * 4^slot * 2^-24 with slot = i (i < 5) or i - 5: no arithmetic beyond the AND
__device__ __forceinline__ uint32_t code_pair(uint32_t w, int i) {
    return i < 5 ? (w & (0x00030003u << (2 * i))) : ((w >> 10) & (0x00030003u << (2 * (i - 5))));
}
__device__ __forceinline__ int code_slot(int i) { return i < 5 ? i : i - 5; }

// stage index and phase parity of ring use number `it` (ring depth ns: 4 unless the planes are large)
__device__ __forceinline__ int ring_slot(int it, int ns) { return ns == 4 ? (it & 3) : it % ns; }
__device__ __forceinline__ uint32_t ring_phase(int it, int ns) { return (uint32_t)(ns == 4 ? (it >> 2) : it / ns) & 1u; }

// KOUT: outliers per K vector known at compile time (static, unrolled splice) or -1 (runtime).
//
// Every MMA is m16n8k16 fp16 with the 2-bit codes as the A operand: a code field masked in place is an
// fp16 subnormal, code * 4^slot * 2^-24, exact and without an offset.  N = 8 columns are the query heads
// of the kv head (GQA <= 8).
//   logits   S^T[token][head]  = codes[token][ch] . (q * 2^e_k)[ch][head]      (2 m-tiles x 8 k-steps)
//                              + delta[token][ch] . q[ch][head]                (sidecar tile, same shape)
//                              + zp[ch] . q[ch][head]                          (one row, broadcast)
//   output   O^T[ch][head]     = codes^T[ch][token] . (P * 2^e_v)[token][head] (8 m-tiles x 2 k-steps, the
//                                16 rows of an m-tile lie in one V scale group)
//                              + vz^T[group][token] . P[token][head]
// The power-of-two factors, zero-points and deltas of a unit are laid out for these fragments by the
// decode warps (the sidecar tile), so the MMA warps multiply and accumulate and do little else.
template <int KOUT, bool WIDE>
__global__ void __launch_bounds__(WarpLayout<WIDE>::THREADS, 1) decode_stage1_kernel(const __grid_constant__ S1Params p) {
    constexpr int NDW = WarpLayout<WIDE>::NDW, NPW = WarpLayout<WIDE>::NPW, PRODUCER_WARP = WarpLayout<WIDE>::PRODUCER_WARP;
    constexpr int S1_THREADS = WarpLayout<WIDE>::THREADS;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // swizzle atoms are 1 KB: align the ring by hand (the launch adds 1 KB of slack)
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int split = blockIdx.x, b = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the first tensor-map copy otherwise pays for fetching its descriptor
    if (threadIdx.x == S1_THREADS - 32 && p.swz != 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&p.tmap_k)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&p.tmap_v)) : "memory");
    }

    // The launch lets this grid start while the kernel before it in the stream is still running (its blocks are
    // placed, shared memory is carved): nothing that kernel may have written - lengths, tables, the query, the
    // planes, the split workspace a previous layer's combine still reads - is touched before this returns.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // ---- split range (same rounding as the reference, paged_decode.py:1428-1432) ----
    const int seq = p.b_seq_len[b];
    if (seq <= 0) return;
    const int per = (((seq + p.S - 1) / p.S) + 31) / 32 * 32;
    const int t0 = split * per;
    const int t1 = min(t0 + per, seq);
    if (t1 <= t0) return;
    const int ntok = t1 - t0;
    int ngroups = (ntok + 31) / 32;
    if (ngroups > MAX_SPLIT_GROUPS || ngroups * p.ppg > MAX_SPLIT_PAGES) {   // host sizing should prevent this
        if (threadIdx.x == 0) or_status(p.status, OMMX_ST_BAD_LENGTH);
        return;
    }
    const int H = p.H, GS = p.GS, NS = p.nstages;
    const int n_iters = (ngroups + GS - 1) / GS;
    const int k_out = KOUT >= 0 ? KOUT : p.k_out;
    const long long wait_limit = (p.abl & ABL_TEST_STALL) ? TEST_WAIT_LIMIT_CYCLES : WAIT_LIMIT_CYCLES;
    // The MMA warps' query words (bf16 pairs) are requested now and turned into operand fragments after the prologue,
    // which hides their round trip behind the table loads: q_s = this lane's 32 consecutive channels (code MMAs),
    // q_d = the channel pairs of the delta MMAs' fragments.  Column n = lane / 4 of every MMA is query head n.
    uint32_t q_s[16], q_d[16];
    if (warp < NCW) {
        const int hq_ = (warp & (H - 1)) * p.gqa + ((lane >> 2) < p.gqa ? (lane >> 2) : 0), j_ = lane & 3;
        const __nv_bfloat16 *qrow = p.q + (int64_t)b * p.q_sb + (int64_t)hq_ * p.q_sh;
        if (p.q_vec_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const uint4 t = __ldg(reinterpret_cast<const uint4 *>(qrow + 32 * j_) + v);
                q_s[4 * v] = t.x; q_s[4 * v + 1] = t.y; q_s[4 * v + 2] = t.z; q_s[4 * v + 3] = t.w;
            }
#pragma unroll
            for (int r = 0; r < 16; ++r) q_d[r] = __ldg(reinterpret_cast<const uint32_t *>(qrow + 16 * (r >> 1) + 8 * (r & 1) + 2 * j_));
        } else {
            const uint16_t *q16 = reinterpret_cast<const uint16_t *>(qrow);
#pragma unroll
            for (int v = 0; v < 16; ++v) q_s[v] = (uint32_t)__ldg(q16 + 32 * j_ + 2 * v) | ((uint32_t)__ldg(q16 + 32 * j_ + 2 * v + 1) << 16);
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                const int c = 16 * (r >> 1) + 8 * (r & 1) + 2 * j_;
                q_d[r] = (uint32_t)__ldg(q16 + c) | ((uint32_t)__ldg(q16 + c + 1) << 16);
            }
        }
    }

    // ---- shared memory carve-up ----
    uint8_t *s_stage = smem;                                            // nstages * stage_bytes
    uint8_t *s_tiles = s_stage + NS * p.stage_bytes;                    // NCW * DT_BYTES
    int32_t *s_tab = reinterpret_cast<int32_t *>(s_tiles + NCW * DT_BYTES);   // page ids, then group slots
    float *s_lut = reinterpret_cast<float *>(s_tab + MAX_SPLIT_PAGES + MAX_SPLIT_GROUPS);
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(s_lut + 16);         // full[], empty[], tile_full[NCW], tile_empty[NCW][], tile_rows[NCW]
    int32_t *s_abort = reinterpret_cast<int32_t *>(s_bar + 2 * MAX_STAGES + (2 + MAX_STAGES) * NCW);
    CopyDesc *s_desc = reinterpret_cast<CopyDesc *>(s_abort + 4);
    const uint32_t bar_full = smem_u32(s_bar), bar_empty = smem_u32(s_bar + MAX_STAGES);
    const uint32_t bar_tfull = smem_u32(s_bar + 2 * MAX_STAGES), bar_tempty = smem_u32(s_bar + 2 * MAX_STAGES + NCW);
    const uint32_t bar_trows = smem_u32(s_bar + 2 * MAX_STAGES + (1 + MAX_STAGES) * NCW);

    // ---- prologue: LUT, barriers, copy descriptors and the split's page / slot tables, spread over the
    //      whole CTA so that the producer can issue the first stage right after the barrier ----
    if (threadIdx.x < 16) {
        const int c = threadIdx.x;
        const int mi = ((c >> 1) & 3) * 2 + (c & 1);                    // exp*2 + mant
        const float mag = mi == 0 ? 0.f : (mi == 1 ? .5f : (float)(2 + (mi & 1)) * (float)(1 << (mi >> 1)) * 0.25f);
        s_lut[c] = (c & 8) ? -mag : mag;
    }
    {
        // one barrier per thread (56 of them: a single thread's serial inits were a microsecond of every launch)
        const int t = (int)threadIdx.x - 32;
        constexpr int NB_RING = 2 * MAX_STAGES, NB_ALL = NB_RING + (2 + MAX_STAGES) * NCW;
        if (t >= 0 && t < NB_ALL) {
            uint32_t count;
            if (t < MAX_STAGES) count = 1;                                     // full[]
            else if (t < NB_RING) count = 3 * NCW;                             // empty[]: 8 MMA warps + 16 tile halves
            else if (t < NB_RING + NCW) count = 2;                             // tile_full[]: the two halves' deltas scattered
            else if (t < NB_RING + NCW + MAX_STAGES * NCW) count = 1;          // tile_empty[][]
            else count = 2;                                                    // tile_rows[]: the two halves' rows written
            mbar_init(bar_full + 8 * t, count);
            if (t == 0) *s_abort = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    }
    const int cpg = 4 * p.ppg + 6;                                      // copies per group
    const int ncopies = GS * cpg;
    {
        // Copy roles (group-in-stage, plane) are tabulated once; the producer's loop body is then one
        // descriptor load, one table lookup, one multiply-add and one copy per role, with no divergent
        // paths, because that single warp's issue latency bounds how fast stages refill.
        const uint32_t page_b = (uint32_t)p.ps * H;                     // (token, head) rows per page
        const int c = (int)threadIdx.x - 64;                            // threads 64.. build one descriptor each
        if (c >= 0 && c < ncopies) {
            CopyDesc d;
            d.src = nullptr; d.unit = 0; d.dst = 0; d.tbase = 0; d.tmul = 0; d.gi = 0; d.tok0 = 0;
            const int gi = c / cpg, ci = c - gi * cpg;
            d.gi = gi;
            const uint32_t gbo = (uint32_t)gi * p.gb_bytes;
            if (ci < 4 * p.ppg) {
                const int pg = ci >> 2, plane = ci & 3;
                const uint32_t w = plane < 2 ? 32u : (plane == 2 ? 4u : 8u);
                d.src = plane == 0 ? p.k_base : (plane == 1 ? p.v_main : (plane == 2 ? p.v_scale : p.v_zp));
                d.unit = page_b * w;
                d.dst = gbo + (plane == 0 ? 0u : (plane == 1 ? (uint32_t)p.o_vm : (plane == 2 ? (uint32_t)p.o_vs : (uint32_t)p.o_vz)))
                      + (uint32_t)pg * page_b * w;
                d.tbase = pg; d.tmul = p.ppg; d.tok0 = pg * p.ps;
                if (p.swz != 0 && plane < 2) d.gi |= (plane + 1) << 8;
            } else {
                const int gp = ci - 4 * p.ppg;
                const bool on = gp < 2 || (k_out > 0 && (gp >= 4 || p.use_map));
                if (on) {
                    const uint32_t w = gp == 0 ? 128u : (gp == 4 ? 128u * p.nbi : (gp == 5 ? 128u * p.nb : 256u));
                    d.src = gp == 0 ? p.k_scale : (gp == 1 ? p.k_zp : (gp == 2 ? p.k_ms : (gp == 3 ? p.k_mc : (gp == 4 ? p.k_obmp : p.k_oval))));
                    d.unit = (uint32_t)H * w;
                    d.dst = gbo + (uint32_t)(gp == 0 ? p.o_ks : (gp == 1 ? p.o_kz : (gp == 2 ? p.o_ms : (gp == 3 ? p.o_mc : (gp == 4 ? p.o_bm : p.o_ov)))));
                    d.tbase = MAX_SPLIT_PAGES; d.tmul = 1;
                }
            }
            s_desc[c] = d;
        }
        // page ids first (s_tab[0..)), group slots behind them
        const int g0 = p.seg_group_base + t0 / 32;                      // first logical group
        const int npages = (ntok + p.ps - 1) / p.ps;
        const int64_t pg0 = ((int64_t)g0 * 32) / p.ps;
        for (int i = threadIdx.x; i < npages; i += S1_THREADS) {
            int64_t pg = load_index(p.r2t, p.tbl64, (int64_t)b * p.r2t_sb + pg0 + i);
            if (pg < 0 || pg >= p.num_pages) { or_status(p.status, OMMX_ST_BAD_PAGE); pg = 0; }
            s_tab[i] = (int)pg;
        }
        for (int i = S1_THREADS - 1 - (int)threadIdx.x; i < ngroups; i += S1_THREADS) {
            int64_t sl = load_index(p.r2g, p.tbl64, (int64_t)b * p.r2g_sb + g0 + i);
            if (sl < 0 || sl >= p.num_slots) { or_status(p.status, OMMX_ST_BAD_GROUP); sl = 0; }
            s_tab[MAX_SPLIT_PAGES + i] = (int)sl;
        }
    }
    __syncthreads();
    // Stage 2 is launched as a programmatic dependent: it may start its own prologue (residual-row
    // logits, which do not depend on this kernel) as soon as SM resources free up, and waits for this
    // grid to finish before it reads the split partials.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int g = lane >> 2, j = lane & 3;
    const int TS = H * 32;                                          // bytes per token row (all heads)
    const float LOG2E = 1.4426950408889634f;
    const bool no_outlier = (p.abl & ABL_NO_OUTLIER) != 0;
    const int n_items = n_iters * NCW * 2;                          // (iteration, unit, tile half) work items of the decode role

    // ---- one stage of the ring: announce its bytes, issue its copies (producer warp) ----
    uint32_t full_total = 0;                                        // bytes of a stage with GS whole groups
    const int whole_groups = ntok / 32;
    const int pw = warp - PRODUCER_WARP;                            // producer warp index (meaningful for those warps only)
    // `nshare` warps split the copies of a stage, this one taking share `share`; the `lead` among them announces the bytes
    auto issue_stage = [&](int it, int nshare, int share, bool lead) __attribute__((always_inline)) {
        const int s = ring_slot(it, NS);
        const int lg0 = it * GS;
        if (lead) {
            uint32_t total = full_total;
            if (lg0 + GS > whole_groups) {                          // last stage: fewer groups or a partial group
                uint32_t mine = 0;
                for (int c = lane; c < ncopies; c += 32) {
                    const CopyDesc d = s_desc[c];
                    const int lg = lg0 + (d.gi & 0xFF);
                    if (d.unit && lg < ngroups && 32 * lg + d.tok0 < ntok) mine += d.unit;
                }
                total = __reduce_add_sync(0xFFFFFFFFu, mine);
            }
            if (lane == 0) mbar_arrive_expect_tx(bar_full + 8 * s, total);
            __syncwarp();
        }
        // (A copy of another producer warp may land before the announcement: the phase cannot complete without the
        // announcing arrival, and the transaction count may run negative meanwhile.)
        const uint32_t sbase = smem_u32(s_stage + (size_t)s * p.stage_bytes);
        for (int c = lane * nshare + share; c < ncopies; c += 32 * nshare) {
            const CopyDesc d = s_desc[c];
            const int lg = lg0 + (d.gi & 0xFF);
            const int kind = d.gi >> 8;
            if (d.unit && lg < ngroups && 32 * lg + d.tok0 < ntok && !((p.abl & ABL_TEST_STALL) && it == 1)) {
                const int64_t idx = s_tab[d.tbase + lg * d.tmul];
                if (kind == 0) bulk_g2s(sbase + d.dst, d.src + idx * d.unit, d.unit, bar_full + 8 * s);
                else tma_2d_g2s(sbase + d.dst, kind == 1 ? &p.tmap_k : &p.tmap_v, 0, (int32_t)idx * p.rows_per_page, bar_full + 8 * s);
            }
        }
    };
    // The first ring fill is on every CTA's critical path: it goes out before the register budgets are resized.
    // A warp issues a bulk copy only about every 60 cycles and different warps overlap, so in the narrow layout the three
    // decode warps of the producer's warpgroup (idle until the data lands) take a quarter of the first fill each.
    if (warp >= PRODUCER_WARP) {
        for (int c = lane; c < ncopies; c += 32) full_total += s_desc[c].unit;
        full_total = __reduce_add_sync(0xFFFFFFFFu, full_total);
    }
    if constexpr (WIDE) {
        if (warp >= PRODUCER_WARP) issue_stage(0, NPW, pw, pw == 0);
    } else {
        if (warp >= PRODUCER_WARP - 3) issue_stage(0, 4, warp - (PRODUCER_WARP - 3), warp == PRODUCER_WARP);
    }

    // ---- one work item of the decode role: half hf of the sidecar tile of (iteration it, unit) ----
    // Build the sidecar tile of a unit between two uses by its MMA warp.  A tile is built in two
    // halves by two warps at once, because the MMA warp of the unit waits for it: half hf takes K
    // channels 64hf..64hf+63 (lane l: channels 64hf + 2l, +1 - delta columns, zero-points, scale
    // factors) and V tokens 16hf..16hf+15 (lane l: token 16hf + l%16, scale groups 2(l/16), +1).
    // Returns false when a bounded wait ran out.
    auto decode_item = [&](const int n) __attribute__((always_inline)) -> bool {
        const int it = n / (2 * NCW), unit = (n >> 1) % NCW, hf = n & 1;
        const int h = unit & (H - 1), gsel = unit >> p.hshift;       // H is a power of two
        uint8_t *tile = s_tiles + unit * DT_BYTES;
        const int s = ring_slot(it, NS);
        const uint32_t ph = ring_phase(it, NS);
        // The fp32 q.zp sums of this half's 64 channels: lane = (query head of the kv head, block of 8 or 16
        // channels).  The lane's raw query values are requested before the waits below, so that the loads are
        // in flight meanwhile.
        const bool gq8 = p.gqa > 4;                               // 8 heads x 4 blocks of 16, else 4 heads x 8 blocks of 8
        const int zq_head = gq8 ? lane >> 2 : lane >> 3, zq_blk = gq8 ? lane & 3 : lane & 7;
        const int zq_c0 = 64 * hf + zq_blk * (gq8 ? 16 : 8);
        uint4 qv0 = make_uint4(0u, 0u, 0u, 0u), qv1 = make_uint4(0u, 0u, 0u, 0u);
        if (zq_head < p.gqa) {
            const __nv_bfloat16 *qp = p.q + (int64_t)b * p.q_sb + (int64_t)(h * p.gqa + zq_head) * p.q_sh + zq_c0;
            if (p.q_vec_ok) {
                qv0 = __ldg(reinterpret_cast<const uint4 *>(qp));
                if (gq8) qv1 = __ldg(reinterpret_cast<const uint4 *>(qp) + 1);
            } else {
                const uint16_t *q16 = reinterpret_cast<const uint16_t *>(qp);
                auto pair = [&](int i) { return (uint32_t)__ldg(q16 + i) | ((uint32_t)__ldg(q16 + i + 1) << 16); };
                qv0 = make_uint4(pair(0), pair(2), pair(4), pair(6));
                if (gq8) qv1 = make_uint4(pair(8), pair(10), pair(12), pair(14));
            }
        }
        if (!mbar_wait(bar_full + 8 * s, ph, wait_limit)) {
            if (lane == 0) { or_status(p.status, OMMX_ST_TIMEOUT); atomicExch(s_abort, 1); }
            return false;
        }
        const int lg = it * GS + gsel;                           // local group of this unit
        if (lg < ngroups && !(p.abl & ABL_NO_COMPUTE)) {
            // Tile `it` of a unit may be written once the MMA warp has read tile it-1.  Decode warps
            // run up to NS groups ahead and the tiles of one unit are built by different warps, so
            // "tile k was read" events rotate over NS barriers per unit (barrier k % NS, phase
            // k / NS): the newest event a waiter can be missing is then always the one it waits
            // for, never an older phase of the same parity.
            uint8_t *gb = s_stage + (size_t)s * p.stage_bytes + (size_t)gsel * p.gb_bytes;
            const int d0 = 64 * hf + 2 * lane;                   // first of this lane's two channels
            if (it > 0 && !mbar_wait(bar_tempty + 8 * (MAX_STAGES * unit + ring_slot(it - 1, NS)), ring_phase(it - 1, NS), wait_limit)) {
                if (lane == 0) { or_status(p.status, OMMX_ST_TIMEOUT); atomicExch(s_abort, 1); }
                return false;
            }
            bool clamped_any = false;
            const bool splice = k_out > 0 && !no_outlier;
            // ---- first the rows the code MMAs and the softmax read (K factors, q.zp sums, V factors and
            //      zero-points): they are cheap, and the MMA warp starts on them while the deltas are scattered ----
            const uint32_t e2 = *reinterpret_cast<const uint16_t *>(gb + p.o_ks + h * 128 + d0);
            const uint32_t z2 = *reinterpret_cast<const uint32_t *>(gb + p.o_kz + h * 256 + 2 * d0);
            // this lane's entry in the fragment-ordered K factor row
            const uint32_t kf_off = ROW_KF * DT_STRIDE + 64u * (2 * hf + (lane >> 4)) + 32u * ((lane >> 3) & 1) + 8u * (lane & 3) + 2u * ((lane >> 2) & 1);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int e = max((int)(int8_t)(e2 >> (8 * c)), -126);
                bool cl;
                const uint32_t fb = pow2_f16_bits(e, cl);
                clamped_any |= cl;
                *reinterpret_cast<uint16_t *>(tile + kf_off + 4 * c) = (uint16_t)fb;
            }
            {   // q.zp in fp32 from the raw bf16 query, as the reference forms it: 8 (16) products per lane, then the
                // lanes of a head are summed by 3 (2) exchanges
                auto dot4 = [](const uint4 &q, const uint4 &z, float acc) {
                    const uint32_t qw[4] = {q.x, q.y, q.z, q.w}, zw[4] = {z.x, z.y, z.z, z.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        acc = fmaf(__uint_as_float(qw[i] << 16), __uint_as_float(zw[i] << 16), acc);
                        acc = fmaf(__uint_as_float(qw[i] & 0xFFFF0000u), __uint_as_float(zw[i] & 0xFFFF0000u), acc);
                    }
                    return acc;
                };
                const uint8_t *zrow = gb + p.o_kz + h * 256 + 2 * zq_c0;
                float sum = dot4(qv0, *reinterpret_cast<const uint4 *>(zrow), 0.f);
                if (gq8) sum = dot4(qv1, *reinterpret_cast<const uint4 *>(zrow + 16), sum);
                sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
                sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
                if (!gq8) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
                if (zq_blk == 0) reinterpret_cast<float *>(tile + ROW_ZP * DT_STRIDE)[8 * hf + zq_head] = sum;   // heads past gqa: 0
            }
            {   // V side: one token, two scale groups: power-of-two factor and zero-point of each
                const int copy = it & 1;
                const int tk = 16 * hf + (lane & 15), cg0 = 2 * (lane >> 4);
                uint32_t ve = 0x8080u;                               // exponent -128 -> factor 0
                uint32_t vz2 = 0u;
                if (32 * lg + tk < ntok) {
                    ve = *reinterpret_cast<const uint16_t *>(gb + p.o_vs + (tk * H + h) * 4 + cg0);
                    vz2 = *reinterpret_cast<const uint32_t *>(gb + p.o_vz + (tk * H + h) * 8 + 2 * cg0);
                }
                uint8_t *vfr = tile + (ROW_VF + copy) * DT_STRIDE + 64 * ((tk >> 1) & 3) + 8 * hf + 4 * ((tk >> 3) & 1) + 2 * (tk & 1) + 16 * cg0;
                uint8_t *ztr = tile + (ROW_ZT + copy) * DT_STRIDE + 2 * tk + 64 * cg0;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    bool cl;
                    const uint32_t fb = pow2_f16_bits((int)(int8_t)(ve >> (8 * c)), cl);
                    clamped_any |= cl;
                    *reinterpret_cast<uint16_t *>(vfr + 16 * c) = (uint16_t)fb;
                    const float vz = bf16_bits_to_f32(c ? (vz2 >> 16) : (vz2 & 0xFFFFu));
                    *reinterpret_cast<uint16_t *>(ztr + 64 * c) = (uint16_t)f16_bits_sat(vz);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_trows + 8 * unit);
            // ---- then the outlier deltas of this half's columns ----
            if (splice) {
                // clear this half's columns of token rows 0..31 (128 bytes per row)
#pragma unroll
                for (int k2 = 0; k2 < 8; ++k2)
                    *reinterpret_cast<uint4 *>(tile + (4 * k2 + (lane >> 3)) * DT_STRIDE + 128 * hf + 16 * (lane & 7)) = make_uint4(0, 0, 0, 0);
                uint32_t ms2 = 0, mc2 = 0;
                if (p.use_map) {
                    ms2 = *reinterpret_cast<const uint32_t *>(gb + p.o_ms + h * 256 + 2 * d0);
                    mc2 = *reinterpret_cast<const uint32_t *>(gb + p.o_mc + h * 256 + 2 * d0);
                }
                uint2 bm2;
                if (!p.idx7) {
                    bm2 = *reinterpret_cast<const uint2 *>(gb + p.o_bm + h * 512 + 4 * d0);
                } else {
                    // relidx7 (attention/codec.py:91-130 of the reference): k ascending token positions, 7 bits each,
                    // LSB first; the outlier set as a bitmask again, the value stream is shared with that encoding
                    uint32_t m2[2];
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const uint8_t *ip = gb + p.o_bm + (h * 128 + d0 + c) * p.nbi;
                        uint32_t w[5] = {0u, 0u, 0u, 0u, 0u};
                        for (int i = 0; i < p.nbi; ++i) w[i >> 2] |= (uint32_t)ip[i] << (8 * (i & 3));
                        uint32_t bits = 0u;
                        for (int r = 0; r < k_out; ++r) {
                            const int bp = 7 * r;
                            const uint32_t f = __funnelshift_r(w[bp >> 5], w[(bp >> 5) + 1], bp & 31) & 0x7Fu;
                            if (f > 31u) or_status(p.status, OMMX_ST_BAD_GROUP);
                            else bits |= 1u << f;
                        }
                        m2[c] = bits;
                    }
                    bm2 = make_uint2(m2[0], m2[1]);
                }
                uint32_t st[2] = {0, 0}, sth[2] = {0, 0};            // nibble stream of each channel: outliers 0..7, 8..15
                const int nb = KOUT >= 0 ? (KOUT + 1) / 2 : p.nb;
                const uint8_t *ov = gb + p.o_ov + (h * 128 + d0) * nb;          // 2*nb bytes, 2-byte aligned
                if (nb == 3) {
                    const uint32_t w0 = reinterpret_cast<const uint16_t *>(ov)[0], w1 = reinterpret_cast<const uint16_t *>(ov)[1],
                                   w2 = reinterpret_cast<const uint16_t *>(ov)[2];
                    st[0] = w0 | ((w1 & 0xFFu) << 16);
                    st[1] = (w1 >> 8) | (w2 << 8);
                } else if (nb == 4) {
                    const uint2 w = *reinterpret_cast<const uint2 *>(ov);
                    st[0] = w.x; st[1] = w.y;
                } else if (nb == 2) {
                    const uint32_t w = *reinterpret_cast<const uint32_t *>(ov);
                    st[0] = w & 0xFFFFu; st[1] = w >> 16;
                } else if (nb > 4) {
                    // 9..16 outliers: the two channels' streams are 2*nb bytes back to back; read them as
                    // 16-bit pieces into a 128-bit little-endian window and cut it at bit 8*nb
                    uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (i < nb) w[i >> 1] |= (uint32_t) reinterpret_cast<const uint16_t *>(ov)[i] << (16 * (i & 1));
                    const int sh = nb > 4 ? 8 * (nb - 4) : 8;        // 8..32 bits of a stream lie above its first word
                    const uint32_t hmask = sh == 32 ? 0xFFFFFFFFu : ((1u << sh) - 1u);
                    st[0] = w[0]; sth[0] = w[1] & hmask;
                    if (sh == 32) { st[1] = w[2]; sth[1] = w[3]; }
                    else { st[1] = __funnelshift_r(w[1], w[2], sh); sth[1] = __funnelshift_r(w[2], w[3], sh) & hmask; }
                } else {
                    const uint32_t w = *reinterpret_cast<const uint16_t *>(ov);
                    st[0] = w & 0xFFu; st[1] = w >> 8;
                }
                __syncwarp();                                        // the cleared rows before any delta lands in them
                const uint32_t bmv[2] = {bm2.x, bm2.y};
                // The code byte holding this lane's channels, row pz: byte pz*TS + h*32 + d0/4 of the (1 KB aligned)
                // k_base block, with the 16-byte chunk bits XOR-ed by the row's swizzle term.  h*32 + d0/4 splits
                // into a part above bit 7 (added to the row) and a part below (the XOR operand).
                const uint32_t k_hi_rel = (uint32_t)(h >> 2) * 128u;
                const uint8_t *k_hi = gb + k_hi_rel;
                const uint32_t k_lo = (uint32_t)((h & 3) * 32 + (d0 >> 2));
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int e = max((int)(int8_t)(e2 >> (8 * c)), -126);
                    const float sc = __uint_as_float((uint32_t)(e + 127) << 23);
                    const float zp = bf16_bits_to_f32(c ? (z2 >> 16) : (z2 & 0xFFFFu));
                    // delta between the outlier value and the base value it replaces, rounded once
                    float A = sc, Bc = 0.f;                     // shared map: lvl*s + zp - (code*s + zp)
                    if (p.use_map) {
                        const float ms = bf16_bits_to_f32(c ? (ms2 >> 16) : (ms2 & 0xFFFFu));
                        const float mc = bf16_bits_to_f32(c ? (mc2 >> 16) : (mc2 & 0xFFFFu));
                        A = __fdividef(1.f, ms);
                        Bc = mc - zp;
                    }
                    uint32_t bits = bmv[c];
                    const uint32_t stream = st[c], stream_hi = sth[c];
                    (void)stream_hi;
                    const int fsh = 2 * ((d0 & 3) + c);          // bit position of the channel's code in its byte
                    uint8_t *col = tile + 2 * d0 + 2 * c;
                    if (KOUT > 0) {
                        if (__popc(bits) == KOUT) {
                            // Two passes: all gathers (base-code byte, FP4 level) first, then the arithmetic and the
                            // stores.  In one pass every load would have to follow the previous outlier's store in
                            // program order (shared memory may alias), i.e. KOUT load round trips in a row.
                            constexpr int KO = KOUT > 0 ? KOUT : 1;
                            uint32_t pzs[KO], cbs[KO];
                            float lvs[KO];
#pragma unroll
                            for (int r = KO - 1; r >= 0; --r) {
                                const int pz = 31 - __clz(bits);
                                bits ^= 1u << pz;
                                pzs[r] = (uint32_t)pz;
                                lvs[r] = s_lut[((r < 8 ? stream : stream_hi) >> (4 * (r & 7))) & 0xFu];
                                const uint32_t row = (uint32_t)pz * (uint32_t)TS;
                                cbs[r] = k_hi[row + (k_lo ^ (((row + k_hi_rel) >> 3) & p.swz))];
                            }
#pragma unroll
                            for (int r = KO - 1; r >= 0; --r) {
                                const float cf = (float)((cbs[r] >> fsh) & 3u);
                                const float X = fmaf(cf, -sc, fmaf(lvs[r], A, Bc));
                                *reinterpret_cast<uint16_t *>(col + pzs[r] * DT_STRIDE) = (uint16_t)f16_bits_of_bf16_rounded(X);
                            }
                        } else {
                            or_status(p.status, OMMX_ST_BAD_GROUP);   // bitmask and value stream disagree
                        }
                    } else {
                        // any other k: one pass at run time
                        int r = __popc(bits) - 1;
                        while (bits) {
                            const int pz = 31 - __clz(bits);
                            bits ^= 1u << pz;
                            const uint32_t nib = ((r < 8 ? stream : stream_hi) >> (4 * (r & 7))) & 0xFu;
                            --r;
                            const uint32_t row = (uint32_t)pz * (uint32_t)TS;
                            const uint32_t cb = k_hi[row + (k_lo ^ (((row + k_hi_rel) >> 3) & p.swz))];
                            const float cf = (float)((cb >> fsh) & 3u);
                            const float X = fmaf(cf, -sc, fmaf(s_lut[nib], A, Bc));
                            *reinterpret_cast<uint16_t *>(col + pz * DT_STRIDE) = (uint16_t)f16_bits_of_bf16_rounded(X);
                        }
                    }
                }
            }
            if (clamped_any) or_status(p.status, OMMX_ST_SCALE_RANGE);
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tfull + 8 * unit);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + 8 * s);
        return true;
    };

    // ---- roles; each branch starts by resizing its warpgroups' register budget and never rejoins ----
    if constexpr (WIDE) {
        if (warp >= PRODUCER_WARP) asm volatile("setmaxnreg.dec.sync.aligned.u32 " OMMX_REGS_PRODUCER ";");
        else if (warp >= NCW) asm volatile("setmaxnreg.dec.sync.aligned.u32 " OMMX_REGS_DECODE ";");
    } else {
        if (warp >= NCW) asm volatile("setmaxnreg.dec.sync.aligned.u32 " OMMX_REGS_DECODE ";");
    }
    bool producer_alive = true;
    if (warp >= PRODUCER_WARP) {
        // =========================== producer warp(s) ===========================
        for (int it = 1; it < n_iters; ++it) {
            // the first NS fills find their slots fresh
            if (it >= NS && !mbar_wait(bar_empty + 8 * ring_slot(it, NS), ring_phase(it, NS) ^ 1, wait_limit)) {
                if (lane == 0) { or_status(p.status, OMMX_ST_TIMEOUT); atomicExch(s_abort, 1); }
                producer_alive = false;
                break;
            }
            issue_stage(it, NPW, pw, pw == 0);
        }
        if constexpr (WIDE) {
            // with several groups per stage, the epilogue's two CTA-wide barriers
            if (GS > 1) { __syncthreads(); __syncthreads(); }
            return;
        }
        // Narrow layout: with every stage on its way this warp has nothing left to do, while the 15 decode warps share
        // 16 items per iteration: it joins them below for the very last item, so that the last iteration's 16 halves are
        // built side by side.
    }

    // =========================== decode + MMA warps ===========================
    // MMA warp w owns unit w = (group-in-stage, kv head) and its softmax state.  The decode warps are
    // stateless: work item number n goes to decode warp n % NDW (narrow layout: except the last one, the producer's).
    if (warp >= NCW) {
        // =========================== decode warps (narrow layout: and the producer, once it is done) ===========================
        const int dw = warp - NCW;
        const bool is_producer = !WIDE && warp == PRODUCER_WARP;
        if (!is_producer) {
            if (dw < NCW) {           // the first to touch tile dw clears it once (unused rows stay zero)
                uint8_t *t0p = s_tiles + dw * DT_BYTES;
                for (int i = lane; i < DT_BYTES / 4; i += 32) reinterpret_cast<uint32_t *>(t0p)[i] = 0u;
            }
            // every tile is cleared before any half of it is written; the narrow layout's producer learns of it without
            // being waited for
            asm volatile("bar.sync 1, %0;" ::"n"(NDW * 32) : "memory");
            if constexpr (!WIDE) asm volatile("bar.arrive 2, %0;" ::"n"((NDW + 1) * 32) : "memory");
        } else {
            asm volatile("bar.sync 2, %0;" ::"n"((NDW + 1) * 32) : "memory");
        }
        const int n_first = is_producer ? n_items - 1 : dw;
        const int n_end = WIDE ? n_items : (is_producer ? (producer_alive ? n_items : 0) : n_items - 1);
        for (int n = n_first; n < n_end; n += NDW)
            if (!decode_item(n)) break;
        if (GS > 1) { __syncthreads(); __syncthreads(); }          // the epilogue's two CTA-wide barriers (see there)
        return;
    }

    // =========================== MMA warps ===========================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 " OMMX_REGS_MMA ";");
    const int unit = warp;
    const int h = unit & (H - 1), gsel = unit >> p.hshift;
    const uint8_t *tile = s_tiles + unit * DT_BYTES;
    const uint32_t tile_s = smem_u32(tile);
    // Column n = g of every MMA is query head g of this kv head.
    const bool head_ok = g < p.gqa;
    // B fragments of q, fp16.  QS: bf16(q*sm_scale) * 4^-slot for the code MMAs, register r = 8*wi + i holds
    // channels (32j + 16wi + i, + 8), the pair a code word yields in one AND.  QD: plain bf16(q*sm_scale) for
    // the delta MMAs, whose tile columns are channels in natural order.
    uint32_t QS[16], QD[16];
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        const int wi = r >> 3, i = r & 7;
        const int e0 = 16 * wi + i, e1 = e0 + 8;                  // channel 32j + e0 / + e1
        const float f = 1.f / (float)(1 << (2 * code_slot(i)));
        float lo = 0.f, hi = 0.f;
        if (head_ok) {
            lo = bf16_round_f32(bf16_bits_to_f32((q_s[e0 >> 1] >> (16 * (e0 & 1))) & 0xFFFFu) * p.sm_scale) * f;
            hi = bf16_round_f32(bf16_bits_to_f32((q_s[e1 >> 1] >> (16 * (e1 & 1))) & 0xFFFFu) * p.sm_scale) * f;
        }
        QS[r] = pack_f16x2(lo, hi);
    }
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        float lo = 0.f, hi = 0.f;
        if (head_ok) {
            lo = bf16_round_f32(bf16_bits_to_f32(q_d[r] & 0xFFFFu) * p.sm_scale);
            hi = bf16_round_f32(bf16_bits_to_f32(q_d[r] >> 16) * p.sm_scale);
        }
        QD[r] = pack_f16x2(lo, hi);
    }
    // per-lane fragment addresses inside the sidecar tile
    const uint32_t a_delta = tile_s + ((lane & 7) + 8 * ((lane >> 3) & 1)) * DT_STRIDE + 16 * (lane >> 4);
    const uint8_t *p_kf = tile + ROW_KF * DT_STRIDE + 64 * j;
    // ---- online softmax state of heads 2j and 2j+1 (the two columns this lane holds) ----
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    // acc[2*cg + u]: rows = channels 32cg + 4g + u (regs 0,1) and 32cg + 4g + 2 + u (regs 2,3), columns = heads
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
    float accz[4] = {0.f, 0.f, 0.f, 0.f};        // rows = V scale groups: sum_t vz[t][cg] * P[t][head]
    uint32_t consumed = 0;
    const bool do_k = !(p.abl & ABL_NO_K), do_v = !(p.abl & ABL_NO_V);
    const bool has_delta = !(k_out == 0 || no_outlier);

    for (int it = 0; it < n_iters; ++it) {
        const int s = ring_slot(it, NS);
        const uint32_t ph = ring_phase(it, NS);
        const int lg = it * GS + gsel;                               // local group of this warp
        const bool active = lg < ngroups && !(p.abl & ABL_NO_COMPUTE);
        if (!mbar_wait(bar_full + 8 * s, ph, wait_limit)) {
            if (lane == 0) { or_status(p.status, OMMX_ST_TIMEOUT); atomicExch(s_abort, 1); }
            m_run[0] = m_run[1] = -INFINITY; l_run[0] = l_run[1] = 0.f;
            break;
        }
        if (active) {
            uint8_t *gb = s_stage + (size_t)s * p.stage_bytes + (size_t)gsel * p.gb_bytes;
            const uint8_t *vreg = gb + p.o_vm;                      // v_main region of the group (1 KB aligned)

            // ======================= logits =======================
            // code words of this lane's four token rows (tokens 8*nt + g), channels 32j..32j+31
            uint2 kw[4];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                kw[nt] = make_uint2(0u, 0u);
                if (do_k) kw[nt] = *reinterpret_cast<const uint2 *>(gb + swz128((uint32_t)((8 * nt + g) * TS + h * 32 + 8 * j), p.swz));
            }
            // The unit's sidecar tile arrives in two steps: first the factor and zero-point rows, then the outlier
            // deltas.  The code MMAs run on the first, while the decode warps still scatter the deltas.
            if (!mbar_wait(bar_trows + 8 * unit, consumed & 1u, wait_limit)) {
                if (lane == 0) { or_status(p.status, OMMX_ST_TIMEOUT); atomicExch(s_abort, 1); }
                m_run[0] = m_run[1] = -INFINITY; l_run[0] = l_run[1] = 0.f;
                break;
            }
            float Sc[2][4], Sd[2][4], Sz[2];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) { Sc[mt][0] = Sc[mt][1] = Sc[mt][2] = Sc[mt][3] = 0.f; Sd[mt][0] = Sd[mt][1] = Sd[mt][2] = Sd[mt][3] = 0.f; }
            // Two accumulators take turns, so that neighbours in the instruction stream never wait on each other
            // (the asm statements keep their order, so the order written here is the order issued).
            {
                // q.zp of heads 2j and 2j+1: the two channel halves' fp32 partial sums, times sm_scale
                const float2 za = *reinterpret_cast<const float2 *>(tile + ROW_ZP * DT_STRIDE + 8 * j);
                const float2 zb = *reinterpret_cast<const float2 *>(tile + ROW_ZP * DT_STRIDE + 32 + 8 * j);
                Sz[0] = (za.x + zb.x) * p.sm_scale;
                Sz[1] = (za.y + zb.y) * p.sm_scale;
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int wi = q >> 2, i0 = 2 * (q & 3);
                    const uint2 fq = reinterpret_cast<const uint2 *>(p_kf)[q];      // this k-step's two factor pairs
                    const uint32_t b0 = hmul2_f16(QS[2 * q], fq.x), b1 = hmul2_f16(QS[2 * q + 1], fq.y);
                    {
                        const uint32_t wlo = wi ? kw[0].y : kw[0].x, whi = wi ? kw[1].y : kw[1].x;
                        mma_f16(Sc[0], code_pair(wlo, i0), code_pair(whi, i0), code_pair(wlo, i0 + 1), code_pair(whi, i0 + 1), b0, b1);
                    }
                    {
                        const uint32_t wlo = wi ? kw[2].y : kw[2].x, whi = wi ? kw[3].y : kw[3].x;
                        mma_f16(Sc[1], code_pair(wlo, i0), code_pair(whi, i0), code_pair(wlo, i0 + 1), code_pair(whi, i0 + 1), b0, b1);
                    }
                }
            }
            if (has_delta) {
                if (!mbar_wait(bar_tfull + 8 * unit, consumed & 1u, wait_limit)) {
                    if (lane == 0) { or_status(p.status, OMMX_ST_TIMEOUT); atomicExch(s_abort, 1); }
                    m_run[0] = m_run[1] = -INFINITY; l_run[0] = l_run[1] = 0.f;
                    break;
                }
                uint32_t d0f[4], d1f[4];                         // delta fragments of m-tile 0 / 1
                ldsm_x4(a_delta, d0f[0], d0f[1], d0f[2], d0f[3]);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    ldsm_x4(a_delta + 16 * DT_STRIDE + 32 * q, d1f[0], d1f[1], d1f[2], d1f[3]);
                    mma_f16(Sd[0], d0f[0], d0f[1], d0f[2], d0f[3], QD[2 * q], QD[2 * q + 1]);
                    if (q < 7) ldsm_x4(a_delta + 32 * (q + 1), d0f[0], d0f[1], d0f[2], d0f[3]);
                    mma_f16(Sd[1], d1f[0], d1f[1], d1f[2], d1f[3], QD[2 * q], QD[2 * q + 1]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * (MAX_STAGES * unit + ring_slot((int)consumed, NS)));   // the next tile may be built
            ++consumed;

            // ======================= online softmax =======================
            // x[mt][r]: token 16mt + g + 8(r>>1), head 2j + (r&1)
            float x[2][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int r = 0; r < 4; ++r) x[mt][r] = fmaf(Sc[mt][r], 1048576.f, Sd[mt][r] + Sz[r & 1]);
            if (p.logit_cap > 0.f) {
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int r = 0; r < 4; ++r) x[mt][r] = p.logit_cap * tanhf(x[mt][r] / p.logit_cap);
            }
            const int tok_base = 32 * lg;
            if (tok_base + 32 > ntok) {
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int r = 0; r < 4; ++r)
                        if (tok_base + 16 * mt + g + 8 * (r >> 1) >= ntok) x[mt][r] = -INFINITY;
            }
            float corr[2], mneg[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                float mloc = fmaxf(fmaxf(x[0][hh], x[0][2 + hh]), fmaxf(x[1][hh], x[1][2 + hh]));
                mloc = fmaxf(mloc, __shfl_xor_sync(0xFFFFFFFFu, mloc, 4));
                mloc = fmaxf(mloc, __shfl_xor_sync(0xFFFFFFFFu, mloc, 8));
                mloc = fmaxf(mloc, __shfl_xor_sync(0xFFFFFFFFu, mloc, 16));
                const float m_new = fmaxf(m_run[hh], mloc);
                const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
                corr[hh] = fast_exp2((m_run[hh] - m_use) * LOG2E);   // m_run = -inf -> 0
                mneg[hh] = -m_use * LOG2E;
                m_run[hh] = m_new;
            }
            float pr[2][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int r = 0; r < 4; ++r) pr[mt][r] = fast_exp2(fmaf(x[mt][r], LOG2E, mneg[r & 1]));
#pragma unroll
            for (int hh = 0; hh < 2; ++hh)
                l_run[hh] = l_run[hh] * corr[hh] + ((pr[0][hh] + pr[0][2 + hh]) + (pr[1][hh] + pr[1][2 + hh]));   // this lane's tokens only
            if (__any_sync(0xFFFFFFFFu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
                for (int i = 0; i < 8; ++i) { acc[i][0] *= corr[0]; acc[i][1] *= corr[1]; acc[i][2] *= corr[0]; acc[i][3] *= corr[1]; }
                accz[0] *= corr[0]; accz[1] *= corr[1];
            }
            // P^T as B fragments: transpose each 8x8 (token, head) block; T[ks][b] = tokens 16ks + 8b + 2j, +1 of head g
            uint32_t T[2][2];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                T[mt][0] = movmatrix_trans(pack_f16x2(pr[mt][0], pr[mt][1]));
                T[mt][1] = movmatrix_trans(pack_f16x2(pr[mt][2], pr[mt][3]));
            }

            // ======================= P.V =======================
            if (do_v) {
                const int copy = it & 1;
                uint32_t VF[16];                                     // factor pairs, index 4cg + 2ks + b
                {
                    const uint8_t *p_vf = tile + (ROW_VF + copy) * DT_STRIDE + 64 * j;
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        const uint4 t = reinterpret_cast<const uint4 *>(p_vf)[v];
                        VF[4 * v] = t.x; VF[4 * v + 1] = t.y; VF[4 * v + 2] = t.z; VF[4 * v + 3] = t.w;
                    }
                }
                const uint8_t *p_zt = tile + (ROW_ZT + copy) * DT_STRIDE + 64 * (g & 3) + 4 * j;
                const uint32_t v_hi_rel = (uint32_t)(h >> 2) * 128u, v_lo = (uint32_t)((h & 3) * 32 + g);
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
                    const int tA = 16 * ks + 2 * j;
                    // Byte 8cg + g of a token row's 32-byte head slice, four scale groups per row.  The swizzle term
                    // of a row only touches bits 4..6, so two XORs give the addresses of groups 0 and 2 and the
                    // other two are 8 bytes on.
                    uint32_t vb[4][4];                               // [token of (tA, tA+1, tA+8, tA+9)][scale group]
#pragma unroll
                    for (int tt = 0; tt < 4; ++tt) {
                        const uint32_t rowhi = (uint32_t)(tA + (tt & 1) + 8 * (tt >> 1)) * (uint32_t)TS + v_hi_rel;
                        const uint32_t tm = (rowhi >> 3) & p.swz;
                        const uint8_t *r0 = vreg + (rowhi + (v_lo ^ tm)), *r1 = vreg + (rowhi + ((v_lo ^ 16u) ^ tm));
                        vb[tt][0] = r0[0]; vb[tt][1] = r0[8];
                        vb[tt][2] = r1[0]; vb[tt][3] = r1[8];
                    }
#pragma unroll
                    for (int cg = 0; cg < 4; ++cg) {
                        // channels 32cg + 4g .. + 3 of four tokens: one byte each
                        const uint32_t bA = vb[0][cg], bA1 = vb[1][cg], bB = vb[2][cg], bB1 = vb[3][cg];
                        const uint32_t w01 = bA | (bA1 << 16), w89 = bB | (bB1 << 16);
                        const uint32_t pb0 = hmul2_f16(T[ks][0], VF[4 * cg + 2 * ks]), pb1 = hmul2_f16(T[ks][1], VF[4 * cg + 2 * ks + 1]);
#pragma unroll
                        for (int u = 0; u < 2; ++u)
                            mma_f16(acc[2 * cg + u], w01 & (0x00030003u << (2 * u)), w01 & (0x00030003u << (2 * u + 4)),
                                    w89 & (0x00030003u << (2 * u)), w89 & (0x00030003u << (2 * u + 4)), pb0, pb1);
                    }
                    uint32_t za0 = 0u, za2 = 0u;
                    if (g < 4) {
                        za0 = *reinterpret_cast<const uint32_t *>(p_zt + 32 * ks);
                        za2 = *reinterpret_cast<const uint32_t *>(p_zt + 32 * ks + 16);
                    }
                    mma_f16(accz, za0, 0u, za2, 0u, T[ks][0], T[ks][1]);
                }
            }
        }
        // release the stage
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + 8 * s);
    }

    // ---- epilogue: this lane holds 16 channels of heads 2j and 2j+1; merge warps that share a head ----
    float l_tot[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        float l = l_run[hh];
        l += __shfl_xor_sync(0xFFFFFFFFu, l, 4);
        l += __shfl_xor_sync(0xFFFFFFFFu, l, 8);
        l += __shfl_xor_sync(0xFFFFFFFFu, l, 16);
        l_tot[hh] = l;
    }
    // outv[hh][4cg + c]: channel 32cg + 4g + c of head 2j + hh, un-normalised
    float outv[2][16];
#pragma unroll
    for (int cg = 0; cg < 4; ++cg) {
        const float bz0 = __shfl_sync(0xFFFFFFFFu, accz[0], 4 * cg + j);
        const float bz1 = __shfl_sync(0xFFFFFFFFu, accz[1], 4 * cg + j);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int u = c & 1, v = c >> 1;
            const float f = 1048576.f / (float)(1 << (2 * c));       // 2^(24 - FBIAS) * 4^-slot
            outv[0][4 * cg + c] = fmaf(acc[2 * cg + u][2 * v], f, bz0);
            outv[1][4 * cg + c] = fmaf(acc[2 * cg + u][2 * v + 1], f, bz1);
        }
    }

    // Several groups per stage (fewer than 8 local kv heads): the warps that share a head merge through the ring memory,
    // once every warp (and the producer) is done with it.  With 8 heads every warp owns its head and writes straight away.
    float *scratch = reinterpret_cast<float *>(s_stage);             // [NCW][32 lanes][36]
    if (GS > 1) {
        __syncthreads();
        if (gsel > 0) {
            float *my = scratch + ((size_t)unit * 32 + lane) * 36;
            my[0] = m_run[0]; my[1] = m_run[1]; my[2] = l_tot[0]; my[3] = l_tot[1];
#pragma unroll
            for (int i = 0; i < 16; ++i) { my[4 + i] = outv[0][i]; my[20 + i] = outv[1][i]; }
        }
        __syncthreads();
    }
    if (gsel == 0) {
        for (int o = 1; o < GS; ++o) {
            const float *ot = scratch + ((size_t)(o * H + h) * 32 + lane) * 36;
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const float m2 = ot[hh], l2 = ot[2 + hh];
                const float mn = fmaxf(m_run[hh], m2);
                const float mu = (mn == -INFINITY) ? 0.f : mn;
                const float c1 = fast_exp2((m_run[hh] - mu) * LOG2E), c2 = fast_exp2((m2 - mu) * LOG2E);
                l_tot[hh] = l_tot[hh] * c1 + l2 * c2;
#pragma unroll
                for (int i = 0; i < 16; ++i) outv[hh][i] = outv[hh][i] * c1 + ot[4 + 16 * hh + i] * c2;
                m_run[hh] = mn;
            }
        }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int head = 2 * j + hh;
            if (head < p.gqa) {
                const float inv = l_tot[hh] > 0.f ? 1.f / l_tot[hh] : 0.f;
                float *dst = p.al + (int64_t)b * p.al_sb + (int64_t)(h * p.gqa + head) * p.al_sh + (int64_t)split * p.al_ss;
#pragma unroll
                for (int cg = 0; cg < 4; ++cg)
#pragma unroll
                    for (int c = 0; c < 4; ++c) dst[32 * cg + 4 * g + c] = outv[hh][4 * cg + c] * inv;
                if (g == 0) dst[HD] = l_tot[hh] > 0.f ? m_run[hh] + logf(l_tot[hh]) : -INFINITY;
            }
        }
    }
}

// =================================================================================================
// Stage 2: bf16 sink/recent rows + log-sum-exp combine (reference: paged_decode.py:2366-2500)
// =================================================================================================
struct S2Params {
    const __nv_bfloat16 *q;
    int64_t q_sb, q_sh;
    int32_t Hq, gqa, D;
    const __nv_bfloat16 *k_tail, *v_tail;
    int64_t t_sb, t_st, t_sh;
    const int32_t *b_tail_len, *b_seq_len;
    int32_t max_tail;
    const float *al;
    int64_t al_sb, al_sh, al_ss;
    int32_t S;
    void *o;
    int32_t o_bf16;
    int64_t o_sb, o_sh;
    float *lse;
    int64_t lse_sb;
    float sm_scale, logit_cap;
    // head-output exchange (g_world <= 1: none)
    int32_t g_world, g_rank;
    uint64_t *const *g_recv;
    float *g_out;
    uint32_t *g_state;
    int32_t *status;
};

constexpr int S2_THREADS = 512;
constexpr int S2_WARPS = S2_THREADS / 32;
constexpr int S2_MAX_TAIL = 256;
constexpr int S2_MAX_SPLITS = 1024;

// One CTA per (query head, sequence).  Warps stripe over the bf16 residual rows for the logits,
// then over the splits for the combine; every loop keeps many independent loads in flight,
// because this kernel is pure latency (a few hundred KB through L2).
__global__ void __launch_bounds__(S2_THREADS) decode_stage2_kernel(const S2Params p) {
    __shared__ float s_q[HD];
    __shared__ float s_logit[S2_MAX_TAIL];
    __shared__ float s_w[S2_MAX_SPLITS];
    __shared__ float s_red[S2_WARPS];
    __shared__ float s_acc[S2_WARPS][HD];
    // the next kernel in the stream (the following layer's stage 1) may be placed as SMs free up; it waits for
    // this grid to finish before it touches memory
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int hq = blockIdx.x, b = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = hq / p.gqa;
    const int seq = p.b_seq_len[b];
    int tail = p.b_tail_len ? p.b_tail_len[b] : 0;
    tail = max(0, min(tail, min(p.max_tail, S2_MAX_TAIL)));
    const int D = p.D;                                                   // == HD
    const int per = (seq > 0 && p.S > 0) ? (((seq + p.S - 1) / p.S) + 31) / 32 * 32 : 0;
    const int nsplit = per > 0 ? min(p.S, (seq + per - 1) / per) : 0;    // splits s with s*per < seq
    const float *base = p.al + (int64_t)b * p.al_sb + (int64_t)hq * p.al_sh;

    constexpr int PRE_T = 5, PRE_S = 10;                                 // rows / splits per warp held in registers
    // ---- bf16 residual rows: logits of this q head (independent of stage 1) ----
    // The K rows of this warp (rows warp, warp+16, ...) are requested together, before the query is in shared memory:
    // this part runs after stage 1 whenever stage 1 fills every SM, so each round trip saved is a round trip per layer.
    if (tail > 0) {
        const __nv_bfloat16 *kt = p.k_tail + (int64_t)b * p.t_sb + (int64_t)kvh * p.t_sh;
        uint2 kpre[PRE_T];
#pragma unroll
        for (int k = 0; k < PRE_T; ++k) {
            const int r = warp + k * S2_WARPS;
            kpre[k] = make_uint2(0u, 0u);
            if (r < tail) kpre[k] = *reinterpret_cast<const uint2 *>(kt + (int64_t)r * p.t_st + 4 * lane);
        }
        if (tid < D) s_q[tid] = __bfloat162float(p.q[(int64_t)b * p.q_sb + (int64_t)hq * p.q_sh + tid]);
        __syncthreads();
        const float q0 = s_q[4 * lane], q1 = s_q[4 * lane + 1], q2 = s_q[4 * lane + 2], q3 = s_q[4 * lane + 3];
        auto logit_of = [&](const uint2 kv) {
            float d = q0 * bf16_bits_to_f32(kv.x & 0xFFFFu) + q1 * bf16_bits_to_f32(kv.x >> 16)
                    + q2 * bf16_bits_to_f32(kv.y & 0xFFFFu) + q3 * bf16_bits_to_f32(kv.y >> 16);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xFFFFFFFFu, d, o);
            float x = d * p.sm_scale;
            if (p.logit_cap > 0.f) x = p.logit_cap * tanhf(x / p.logit_cap);
            return x;
        };
#pragma unroll
        for (int k = 0; k < PRE_T; ++k) {
            const int r = warp + k * S2_WARPS;
            if (r < tail) {                                              // warp-uniform
                const float x = logit_of(kpre[k]);
                if (lane == 0) s_logit[r] = x;
            }
        }
        for (int r = warp + PRE_T * S2_WARPS; r < tail; r += S2_WARPS) {
            const float x = logit_of(*reinterpret_cast<const uint2 *>(kt + (int64_t)r * p.t_st + 4 * lane));
            if (lane == 0) s_logit[r] = x;
        }
    }
    // residual V rows of this warp (rows warp, warp+16, ...), requested before the wait below: they do not depend on stage 1
    const __nv_bfloat16 *vt = p.v_tail + (int64_t)b * p.t_sb + (int64_t)kvh * p.t_sh;
    uint32_t vpre[PRE_T][4];                                             // raw bf16 bits: turned into floats where they are used
#pragma unroll
    for (int k = 0; k < PRE_T; ++k) {
        const int r = warp + k * S2_WARPS;
        vpre[k][0] = vpre[k][1] = vpre[k][2] = vpre[k][3] = 0u;
        if (r < tail) {
            const uint16_t *row = reinterpret_cast<const uint16_t *>(vt + (int64_t)r * p.t_st);
            vpre[k][0] = row[lane]; vpre[k][1] = row[lane + 32]; vpre[k][2] = row[lane + 64]; vpre[k][3] = row[lane + 96];
        }
    }
    // ---- everything below reads what stage 1 wrote: wait for that grid (no-op without a
    //      programmatic launch) ----
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // Every warp folds its own splits (warp, warp+16, ...) and its own residual rows into a private softmax state -
    // maximum, sum of weights, weighted rows - with no exchange: the lse of a split is read by all lanes at once (one
    // address), the residual logits of rows warp, warp+16, ... were written by this very warp.  The 16 states are
    // merged once at the end.  The split rows are requested together with the lse values, not after the weights are
    // known: the kernel is a chain of global round trips and this takes one link out of it.
    float spre[PRE_S][4], lpre[PRE_S];
#pragma unroll
    for (int k = 0; k < PRE_S; ++k) {
        const int s = warp + k * S2_WARPS;
        spre[k][0] = spre[k][1] = spre[k][2] = spre[k][3] = 0.f;
        lpre[k] = -INFINITY;
        if (s < nsplit) {
            const float *row = base + (int64_t)s * p.al_ss;
            spre[k][0] = row[lane]; spre[k][1] = row[lane + 32]; spre[k][2] = row[lane + 64]; spre[k][3] = row[lane + 96];
            lpre[k] = row[D];
        }
    }
    __syncwarp();                                                        // s_logit rows of this warp (lane 0 wrote them)
    float m_w = -INFINITY;
#pragma unroll
    for (int k = 0; k < PRE_S; ++k) m_w = fmaxf(m_w, lpre[k]);
    for (int s = warp + PRE_S * S2_WARPS; s < nsplit; s += S2_WARPS) m_w = fmaxf(m_w, base[(int64_t)s * p.al_ss + D]);
    for (int r = warp; r < tail; r += S2_WARPS) m_w = fmaxf(m_w, s_logit[r]);
    const float m_safe = (m_w == -INFINITY) ? 0.f : m_w;
    // weighted sum: lane owns channels lane + 32*i
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, den_w = 0.f;
#pragma unroll
    for (int k = 0; k < PRE_S; ++k) {
        const float w = __expf(lpre[k] - m_safe);                        // exp(-inf) = 0 for the slots past nsplit
        den_w += w;
        a0 += w * spre[k][0]; a1 += w * spre[k][1]; a2 += w * spre[k][2]; a3 += w * spre[k][3];
    }
#pragma unroll 4
    for (int s = warp + PRE_S * S2_WARPS; s < nsplit; s += S2_WARPS) {
        const float *row = base + (int64_t)s * p.al_ss;
        const float w = __expf(row[D] - m_safe);
        den_w += w;
        a0 += w * row[lane]; a1 += w * row[lane + 32]; a2 += w * row[lane + 64]; a3 += w * row[lane + 96];
    }
    if (tail > 0) {
#pragma unroll
        for (int k = 0; k < PRE_T; ++k) {
            const int r = warp + k * S2_WARPS;
            if (r < tail) {
                const float w = __expf(s_logit[r] - m_safe);
                den_w += w;
                a0 += w * bf16_bits_to_f32(vpre[k][0]); a1 += w * bf16_bits_to_f32(vpre[k][1]);
                a2 += w * bf16_bits_to_f32(vpre[k][2]); a3 += w * bf16_bits_to_f32(vpre[k][3]);
            }
        }
#pragma unroll 4
        for (int r = warp + PRE_T * S2_WARPS; r < tail; r += S2_WARPS) {
            const __nv_bfloat16 *row = vt + (int64_t)r * p.t_st;
            const float w = __expf(s_logit[r] - m_safe);
            den_w += w;
            a0 += w * __bfloat162float(row[lane]); a1 += w * __bfloat162float(row[lane + 32]);
            a2 += w * __bfloat162float(row[lane + 64]); a3 += w * __bfloat162float(row[lane + 96]);
        }
    }
    s_acc[warp][lane] = a0; s_acc[warp][lane + 32] = a1;
    s_acc[warp][lane + 64] = a2; s_acc[warp][lane + 96] = a3;
    if (lane == 0) { s_red[warp] = m_w; s_w[warp] = den_w; }
    __syncthreads();
    // ---- merge of the 16 states ----
    float out = 0.f;
    if (tid < D) {
        float g_max = s_red[0];
#pragma unroll
        for (int w = 1; w < S2_WARPS; ++w) g_max = fmaxf(g_max, s_red[w]);
        const float g_safe = (g_max == -INFINITY) ? 0.f : g_max;
        float acc = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < S2_WARPS; ++w) {
            const float e = __expf(s_red[w] - g_safe);                   // 0 for a warp that saw nothing
            acc = fmaf(s_acc[w][tid], e, acc);
            den = fmaf(s_w[w], e, den);
        }
        out = acc / (den > 0.f ? den : 1.f);
        if (p.o_bf16) reinterpret_cast<__nv_bfloat16 *>(p.o)[(int64_t)b * p.o_sb + (int64_t)hq * p.o_sh + tid] = __float2bfloat16_rn(out);
        else reinterpret_cast<float *>(p.o)[(int64_t)b * p.o_sb + (int64_t)hq * p.o_sh + tid] = out;
        if (tid == 0) p.lse[(int64_t)b * p.lse_sb + hq] = g_max + logf(den);
    }
    if (p.g_world > 1) {
        // Sharded heads: the row travels to every peer as 8-byte words (value, call count); a word arrives whole,
        // so the count tells the receiver that the value beside it is this call's.  Then this block collects the
        // same row of every peer from its own receive buffer.
        __shared__ uint32_t s_epoch;
        if (tid == 0) s_epoch = *reinterpret_cast<volatile uint32_t *>(&p.g_state[0]) + 1u;
        __syncthreads();
        const uint32_t epoch = s_epoch;
        const int64_t slot = (int64_t)gridDim.y * p.Hq * D;            // elements of one rank's slot
        const int64_t row = ((int64_t)b * p.Hq + hq) * D;
        if (tid < D) {
            const uint64_t word = ((uint64_t)epoch << 32) | (uint64_t)__float_as_uint(out);
            for (int r = 0; r < p.g_world; ++r)
                if (r != p.g_rank)
                    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p.g_recv[r] + (int64_t)p.g_rank * slot + row + tid), "l"(word) : "memory");
            p.g_out[(int64_t)p.g_rank * slot + row + tid] = out;
        }
        const uint64_t *mine = p.g_recv[p.g_rank];
        const long long t_end = clock64() + WAIT_LIMIT_CYCLES;
        const int n_words = (p.g_world - 1) * D;
        // two words per thread and round, both requested before either is looked at
        for (int idx = tid; idx < n_words; idx += 2 * S2_THREADS) {
            const uint64_t *src[2];
            float *dst[2];
            bool pending[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int i = idx + u * S2_THREADS;
                pending[u] = i < n_words;
                int r = pending[u] ? i / D : 0;
                const int e = pending[u] ? i - r * D : 0;
                r += (r >= p.g_rank) ? 1 : 0;                          // skip the own slot
                src[u] = mine + (int64_t)r * slot + row + e;
                dst[u] = p.g_out + (int64_t)r * slot + row + e;
            }
            for (uint32_t i = 1; pending[0] || pending[1]; ++i) {
                uint64_t word[2] = {0, 0};
#pragma unroll
                for (int u = 0; u < 2; ++u)
                    if (pending[u]) asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(word[u]) : "l"(src[u]) : "memory");
#pragma unroll
                for (int u = 0; u < 2; ++u)
                    if (pending[u] && (uint32_t)(word[u] >> 32) == epoch) {
                        *dst[u] = __uint_as_float((uint32_t)word[u]);
                        pending[u] = false;
                    }
                if ((i & 63u) == 0 && clock64() > t_end) { or_status(p.status, OMMX_ST_TIMEOUT); break; }
            }
        }
        // the call count moves on once every block has read it: each block reads it before it draws its ticket
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            const uint32_t t = atomicAdd(&p.g_state[1], 1u);
            if (t == gridDim.x * gridDim.y - 1u) {
                p.g_state[1] = 0u;
                p.g_state[0] = epoch;
            }
        }
    }
}

// =================================================================================================
// merge of partial softmax states (reference: paged_decode.py:2650-2690)
// =================================================================================================
__global__ void __launch_bounds__(128) merge_states_kernel(const float *o_parts, const float *lse_parts,
                                                           const int32_t *valid, int P, int R, int D,
                                                           float *o, float *lse) {
    const int r = blockIdx.x;
    int np = P;
    if (valid) { int v = valid[r]; if (v >= 0) np = min(v, P); }
    float m = -INFINITY;
    for (int q = 0; q < np; ++q) m = fmaxf(m, lse_parts[(int64_t)q * R + r]);
    const float ms = (m == -INFINITY) ? 0.f : m;
    float den = 0.f;
    for (int q = 0; q < np; ++q) den += __expf(lse_parts[(int64_t)q * R + r] - ms);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.f;
        for (int q = 0; q < np; ++q)
            acc += __expf(lse_parts[(int64_t)q * R + r] - ms) * o_parts[((int64_t)q * R + r) * D + d];
        o[(int64_t)r * D + d] = acc / (den > 0.f ? den : 1.f);
    }
    if (threadIdx.x == 0) lse[r] = ms + logf(den);
}

// =================================================================================================
// host side
// =================================================================================================
static int validate_decode(const ommx_decode_args *a) {
    if (!a) return fail(OMMX_E_ARG, "decode: null args");
    const ommx_kv_planes &pl = a->planes;
    if (!a->q || !a->o || !a->lse || !a->attn_logits || !a->b_seq_len)
        return fail(OMMX_E_ARG, "decode: q/o/lse/attn_logits/b_seq_len must not be null");
    if (a->q_dtype != OMMX_DT_BF16) return fail(OMMX_E_UNSUPPORTED, "decode: q must be bf16");
    if (a->o_dtype != OMMX_DT_F32 && a->o_dtype != OMMX_DT_BF16) return fail(OMMX_E_UNSUPPORTED, "decode: o must be f32 or bf16");
    if (pl.head_dim != HD) return fail(OMMX_E_UNSUPPORTED, "decode: head_dim=%d (this build serves %d)", pl.head_dim, HD);
    if (pl.n_kv_heads != 1 && pl.n_kv_heads != 2 && pl.n_kv_heads != 4 && pl.n_kv_heads != 8)
        return fail(OMMX_E_UNSUPPORTED, "decode: n_kv_heads=%d per device must be 1, 2, 4 or 8", pl.n_kv_heads);
    if (a->batch <= 0 || a->n_q_heads <= 0 || a->n_q_heads % pl.n_kv_heads != 0)
        return fail(OMMX_E_ARG, "decode: batch=%d n_q_heads=%d n_kv_heads=%d", a->batch, a->n_q_heads, pl.n_kv_heads);
    if (a->n_q_heads / pl.n_kv_heads > 8)
        return fail(OMMX_E_UNSUPPORTED, "decode: GQA group of %d query heads per kv head (max 8)", a->n_q_heads / pl.n_kv_heads);
    if (pl.page_size != 8 && pl.page_size != 16 && pl.page_size != 32)
        return fail(OMMX_E_UNSUPPORTED, "decode: page_size=%d must be 8, 16 or 32", pl.page_size);
    if (pl.scale_kind != OMMX_SCALE_INT8_EXP)
        return fail(OMMX_E_UNSUPPORTED, "decode: only int8 power-of-two scale planes are served (pack with use_pow2)");
    if (pl.outliers_per_vector < 0 || pl.outliers_per_vector > 16)
        return fail(OMMX_E_UNSUPPORTED, "decode: outliers_per_vector=%d outside [0,16]", pl.outliers_per_vector);
    if (pl.outlier_index != OMMX_OIDX_BITMASK && pl.outlier_index != OMMX_OIDX_RELIDX7)
        return fail(OMMX_E_ARG, "decode: outlier_index=%d", pl.outlier_index);
    if (pl.outlier_index == OMMX_OIDX_RELIDX7 && (128 * ((7 * pl.outliers_per_vector + 7) / 8)) % 16 != 0)
        return fail(OMMX_E_UNSUPPORTED, "decode: relidx7 frames of %d outliers do not stage in 16-byte pieces", pl.outliers_per_vector);
    if (a->packed_start_offset != 0) return fail(OMMX_E_UNSUPPORTED, "decode: packed_start_offset must be 0");
    if (a->seg_group_base < 0) return fail(OMMX_E_ARG, "decode: seg_group_base=%d", a->seg_group_base);
    if (a->num_kv_splits < 1) return fail(OMMX_E_ARG, "decode: num_kv_splits=%d", a->num_kv_splits);
    if (a->num_kv_splits > S2_MAX_SPLITS) return fail(OMMX_E_UNSUPPORTED, "decode: num_kv_splits=%d (max %d)", a->num_kv_splits, S2_MAX_SPLITS);
    if (a->max_tail_len > S2_MAX_TAIL) return fail(OMMX_E_UNSUPPORTED, "decode: max_tail_len=%d (max %d)", a->max_tail_len, S2_MAX_TAIL);
    if (a->max_tail_len > 0 && (!a->k_tail || !a->v_tail || !a->b_tail_len))
        return fail(OMMX_E_ARG, "decode: max_tail_len>0 needs k_tail, v_tail and b_tail_len");
    if (a->max_seq_len > 0) {
        if (!a->req_to_token || !a->req_to_group) return fail(OMMX_E_ARG, "decode: page / group tables are null");
        if (!pl.k_base || !pl.k_scale || !pl.k_zp || !pl.v_main || !pl.v_scale || !pl.v_zp)
            return fail(OMMX_E_ARG, "decode: a KV plane is null");
        if (pl.outliers_per_vector > 0 && (!pl.k_obmp || !pl.k_oval))
            return fail(OMMX_E_ARG, "decode: k>0 needs k_obmp and k_oval");
        if (pl.outliers_per_vector > 0 && pl.kv_outlier_map && (!pl.k_mapscale || !pl.k_mapcenter))
            return fail(OMMX_E_ARG, "decode: kv_outlier_map needs k_mapscale and k_mapcenter");
        const void *pp[] = {pl.k_base, pl.k_scale, pl.k_zp, pl.k_obmp, pl.k_oval, pl.k_mapscale, pl.k_mapcenter,
                            pl.v_main, pl.v_scale, pl.v_zp};
        for (const void *x : pp)
            if (((uintptr_t)x & 15) != 0) return fail(OMMX_E_ARG, "decode: every KV plane must be 16-byte aligned");
        const int min_s = ommx_b200_min_num_kv_splits(a->max_seq_len, pl.page_size);
        if (a->num_kv_splits < min_s)
            return fail(OMMX_E_ARG, "decode: num_kv_splits=%d too small for max_seq_len=%d (need >= %d)",
                        a->num_kv_splits, a->max_seq_len, min_s);
    }
    if (a->al_stride_s < HD + 1) return fail(OMMX_E_ARG, "decode: attn_logits last dim must be head_dim+1");
    return 0;
}

// ---- tensor maps of the code planes (driver entry point looked up at run time, no link dependency) ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static std::atomic<int> state{0};                 // 0 unknown, 1 found, 2 absent
    static EncodeTiledFn fn = nullptr;
    int st = state.load(std::memory_order_acquire);
    if (st == 0) {
        void *f = nullptr;
        cudaDriverEntryPointQueryResult q;
        const bool ok = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
                        q == cudaDriverEntryPointSuccess && f != nullptr;
        if (ok) fn = reinterpret_cast<EncodeTiledFn>(f);
        (void)cudaGetLastError();
        state.store(ok ? 1 : 2, std::memory_order_release);
        st = ok ? 1 : 2;
    }
    return st == 1 ? fn : nullptr;
}

// Plane viewed as [bytes/128][128] uint8, box = one page, 128-byte swizzle.  Returns false when the
// map cannot be built (the caller then stages the plane with plain bulk copies).
// Encoded maps are kept in a small table keyed by (base, bytes, box rows): a serving loop calls with the
// same planes every step and the driver call costs about a microsecond.
static bool make_code_map(CUtensorMap *m, const void *base, int64_t total_bytes, int rows_per_page) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr || total_bytes < 128 || rows_per_page < 8 || rows_per_page > 256) return false;
    // 512 sets x 4 ways, keyed by (device, base, bytes, box rows) and compared in full; a set that is
    // full evicts round-robin.  2048 entries hold the two code planes of a 1000-layer model.
    struct Entry { const void *base; int64_t bytes; int rows, dev; CUtensorMap map; };
    constexpr int SETS = 512, WAYS = 4;
    static Entry table[SETS][WAYS];
    static uint8_t next_way[SETS];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { (void)cudaGetLastError(); return false; }
    const uintptr_t key = reinterpret_cast<uintptr_t>(base) >> 8;
    const size_t set = (size_t)((key ^ (key >> 9) ^ (key >> 18) ^ (uintptr_t)dev * 0x9E37u) % SETS);
    {
        std::lock_guard<std::mutex> g(mu);
        for (int w = 0; w < WAYS; ++w) {
            const Entry &e = table[set][w];
            if (e.base == base && e.bytes == total_bytes && e.rows == rows_per_page && e.dev == dev) { *m = e.map; return true; }
        }
    }
    cuuint64_t gdim[2] = {128, (cuuint64_t)(total_bytes / 128)};
    cuuint64_t gstride[1] = {128};
    cuuint32_t box[2] = {128, (cuuint32_t)rows_per_page};
    cuuint32_t estr[2] = {1, 1};
    if (fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), gdim, gstride, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    std::lock_guard<std::mutex> g(mu);
    Entry &e = table[set][next_way[set]];
    next_way[set] = (uint8_t)((next_way[set] + 1) % WAYS);
    e.base = base; e.bytes = total_bytes; e.rows = rows_per_page; e.dev = dev; e.map = *m;
    return true;
}

static size_t stage1_smem(const S1Params &p) {
    return 1024 + (size_t)p.nstages * p.stage_bytes + (size_t)NCW * DT_BYTES + (MAX_SPLIT_GROUPS + MAX_SPLIT_PAGES) * 4 + 64
           + (2 * MAX_STAGES + (2 + MAX_STAGES) * NCW) * 8 + 16
           + (size_t)p.GS * (4 * p.ppg + 6) * sizeof(CopyDesc);       // the copy roles of one stage come last
}

// Launch as a programmatic dependent of whatever precedes it in the stream: the grid may be placed while that
// kernel drains, and the kernel itself waits (griddepcontrol.wait) before it reads or writes global memory.
template <typename Kernel, typename Params>
static cudaError_t launch_overlapping_previous(Kernel kernel, dim3 grid, int threads, size_t smem, cudaStream_t st, const Params &p) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

constexpr int MAX_DEVICES = 64;
static int current_device(int *dev) {
    OMMX_CUDA_TRY(cudaGetDevice(dev));
    if (*dev < 0 || *dev >= MAX_DEVICES) return fail(OMMX_E_UNSUPPORTED, "device ordinal %d (this build tracks %d devices)", *dev, MAX_DEVICES);
    return 0;
}

template <int KOUT, bool WIDE>
static int launch_s1_layout(const S1Params &p, dim3 grid, size_t smem, cudaStream_t st) {
    using L = WarpLayout<WIDE>;
    // function attributes belong to (kernel instantiation, device): one entry per device ordinal
    static std::atomic<size_t> attr_smem[MAX_DEVICES];
    static std::atomic<int> regs_state[MAX_DEVICES];   // 0 unknown, 1 enough, 2 too few
    int dev = 0;
    if (int rc = current_device(&dev)) return rc;
    int regs_ok = regs_state[dev].load(std::memory_order_acquire);
    if (regs_ok == 0) {
        cudaFuncAttributes fa;
        OMMX_CUDA_TRY(cudaFuncGetAttributes(&fa, decode_stage1_kernel<KOUT, WIDE>));
        // setmaxnreg.inc must find the registers the other roles gave back
        const int need = NCW * 32 * REGS_MMA + (WIDE ? L::NDW * 32 * REGS_DECODE + L::NPW * 32 * REGS_PRODUCER
                                                     : (L::THREADS - NCW * 32) * REGS_DECODE);
        regs_ok = fa.numRegs * L::THREADS >= need ? 1 : 2;
        regs_state[dev].store(regs_ok, std::memory_order_release);
    }
    if (regs_ok != 1) return fail(OMMX_E_CUDA, "stage 1 was compiled with fewer registers than its warp roles need");
    if (smem > attr_smem[dev].load(std::memory_order_acquire)) {
        OMMX_CUDA_TRY(cudaFuncSetAttribute(decode_stage1_kernel<KOUT, WIDE>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_smem[dev].store(smem, std::memory_order_release);
    }
    OMMX_CUDA_TRY(launch_overlapping_previous(decode_stage1_kernel<KOUT, WIDE>, grid, L::THREADS, smem, st, p));
    count_launch();
    return 0;
}
// one or two local kv heads: many small copies per ring stage, the wide layout's four producer warps issue them
template <int KOUT>
static int launch_s1(const S1Params &p, dim3 grid, size_t smem, cudaStream_t st) {
    return p.H <= 2 ? launch_s1_layout<KOUT, true>(p, grid, smem, st) : launch_s1_layout<KOUT, false>(p, grid, smem, st);
}

}  // namespace ommx
#include "ommx_decode_tc.cuh"
namespace ommx {

// Which stage-1 kernel serves a call.  The register-operand kernel (decode_stage1_kernel) is the default: on B200 it
// is the faster of the two (53 us against 142 us per 64K-context layer).  OMMX_B200_STAGE1=tc selects the tensor-core
// kernel (decode_stage1_tc_kernel) where its shared-memory plan fits - 4 or 8 local kv heads with GQA <= 4, fewer
// heads at any GQA <= 8 - and no differential-timing knob is set; it produces the same results within the path's
// tolerance and is kept for further work on its pipeline.  The variable is read per call.
static int stage1_choice() {
    const char *e = getenv("OMMX_B200_STAGE1");
    return (e && !strcmp(e, "tc")) ? 1 : 0;
}

static int launch_stage1(const ommx_decode_args *a, cudaStream_t st) {
    if (a->max_seq_len <= 0) return 0;                                   // tail-only decode
    const ommx_kv_planes &pl = a->planes;
    S1Params p;
    p.q = (const __nv_bfloat16 *)a->q; p.q_sb = a->q_stride_b; p.q_sh = a->q_stride_h;
    p.B = a->batch; p.Hq = a->n_q_heads; p.H = pl.n_kv_heads; p.gqa = a->n_q_heads / pl.n_kv_heads;
    p.q_vec_ok = (((uintptr_t)a->q & 15) == 0 && a->q_stride_b % 8 == 0 && a->q_stride_h % 8 == 0) ? 1 : 0;
    p.k_base = (const uint8_t *)pl.k_base; p.v_main = (const uint8_t *)pl.v_main;
    p.v_scale = (const uint8_t *)pl.v_scale; p.v_zp = (const uint8_t *)pl.v_zp;
    p.k_scale = (const uint8_t *)pl.k_scale; p.k_zp = (const uint8_t *)pl.k_zp;
    p.k_ms = (const uint8_t *)pl.k_mapscale; p.k_mc = (const uint8_t *)pl.k_mapcenter;
    p.k_obmp = (const uint8_t *)pl.k_obmp; p.k_oval = (const uint8_t *)pl.k_oval;
    p.ps = pl.page_size; p.ppg = 32 / pl.page_size; p.num_pages = pl.num_pages; p.num_slots = pl.num_group_slots;
    p.k_out = pl.outliers_per_vector; p.nb = (pl.outliers_per_vector + 1) / 2;
    p.idx7 = (pl.outlier_index == OMMX_OIDX_RELIDX7 && pl.outliers_per_vector > 0) ? 1 : 0;
    p.nbi = p.idx7 ? (7 * pl.outliers_per_vector + 7) / 8 : 4;
    p.use_map = (pl.kv_outlier_map && pl.outliers_per_vector > 0) ? 1 : 0;
    p.b_seq_len = a->b_seq_len; p.r2t = a->req_to_token; p.r2g = a->req_to_group; p.tbl64 = a->table_is_int64;
    p.r2t_sb = a->r2t_stride_b; p.r2g_sb = a->r2g_stride_b;
    p.al = a->attn_logits; p.al_sb = a->al_stride_b; p.al_sh = a->al_stride_h; p.al_ss = a->al_stride_s;
    p.S = a->num_kv_splits; p.seg_group_base = a->seg_group_base;
    p.sm_scale = a->sm_scale; p.logit_cap = a->logit_cap; p.status = a->status;
    const int H = p.H;
    p.GS = NCW / H;
    p.hshift = H == 8 ? 3 : (H == 4 ? 2 : (H == 2 ? 1 : 0));
    p.o_vm = H * 1024; p.o_vs = H * 2048; p.o_vz = p.o_vs + H * 128; p.o_ks = p.o_vz + H * 256;
    p.o_kz = p.o_ks + H * 128; p.o_ms = p.o_kz + H * 256; p.o_mc = p.o_ms + H * 256; p.o_bm = p.o_mc + H * 256;
    p.o_ov = (p.o_bm + H * 128 * p.nbi + 15) / 16 * 16;
    p.gb_bytes = p.o_ov + H * 128 * (p.nb > 0 ? p.nb : 0);
    // swizzled tensor-map staging of the two code planes when a page is whole 1 KB swizzle atoms and
    // the 1 KB rounding of the group block still fits shared memory (4 or 8 local kv heads)
    const int64_t page_bytes = (int64_t)p.ps * H * 32;
    p.swz = 0;
    p.rows_per_page = (int32_t)(page_bytes / 128);
    memset(&p.tmap_k, 0, sizeof(CUtensorMap));
    memset(&p.tmap_v, 0, sizeof(CUtensorMap));
    if (H >= 4 && page_bytes % 1024 == 0 &&
        make_code_map(&p.tmap_k, pl.k_base, (int64_t)pl.num_pages * page_bytes, p.rows_per_page) &&
        make_code_map(&p.tmap_v, pl.v_main, (int64_t)pl.num_pages * page_bytes, p.rows_per_page))
        p.swz = 0x70u;
    const int round_to = p.swz ? 1024 : 128;
    p.gb_bytes = (p.gb_bytes + round_to - 1) / round_to * round_to;
    p.stage_bytes = p.GS * p.gb_bytes;
    p.abl = a->abl_flags;
    if (stage1_choice() == 1 && p.abl == 0 && p.gqa <= 8 && !p.idx7) {
        TcParams T;
        T.s = p;
        T.s.GS = 1;
        T.s.stage_bytes = p.gb_bytes;
        const int gqap = p.gqa <= 4 ? 4 : 8;
        const int per_max = ((a->max_seq_len + a->num_kv_splits - 1) / a->num_kv_splits + 31) / 32;   // groups of the longest split
        const size_t tsmem = tc_layout(T, gqap, per_max + 1);
        if (tsmem != 0 && tsmem <= 232448) {
            dim3 tgrid(a->num_kv_splits, a->batch);
            if (gqap == 4) return H == 8 ? launch_tc<4, true>(T, tgrid, tsmem, st) : launch_tc<4, false>(T, tgrid, tsmem, st);
            return H == 8 ? launch_tc<8, true>(T, tgrid, tsmem, st) : launch_tc<8, false>(T, tgrid, tsmem, st);
        }
    }
    // deepest ring that fits the 227 KB a CTA may use
    p.nstages = MAX_STAGES;
    while (p.nstages > 2 && stage1_smem(p) > 232448) --p.nstages;
    const size_t smem = stage1_smem(p);
    if (smem > 232448) return fail(OMMX_E_UNSUPPORTED, "stage 1 planes of one group do not fit shared memory");
    dim3 grid(a->num_kv_splits, a->batch);
    switch (p.k_out) {                       // the serving recipes get the unrolled two-pass splice
        case 0: return launch_s1<0>(p, grid, smem, st);
        case 2: return launch_s1<2>(p, grid, smem, st);
        case 4: return launch_s1<4>(p, grid, smem, st);
        case 6: return launch_s1<6>(p, grid, smem, st);
        case 8: return launch_s1<8>(p, grid, smem, st);
        case 12: return launch_s1<12>(p, grid, smem, st);
        default: return launch_s1<-1>(p, grid, smem, st);
    }
}

// `after_stage1`: the previous kernel in the stream is this call's own stage 1, so stage 2 may be
// launched as its programmatic dependent.
static int launch_stage2(const ommx_decode_args *a, cudaStream_t st, bool after_stage1 = false) {
    const ommx_kv_planes &pl = a->planes;
    S2Params p;
    p.q = (const __nv_bfloat16 *)a->q; p.q_sb = a->q_stride_b; p.q_sh = a->q_stride_h;
    p.Hq = a->n_q_heads; p.gqa = a->n_q_heads / pl.n_kv_heads; p.D = pl.head_dim;
    p.k_tail = (const __nv_bfloat16 *)a->k_tail; p.v_tail = (const __nv_bfloat16 *)a->v_tail;
    p.t_sb = a->tail_stride_b; p.t_st = a->tail_stride_t; p.t_sh = a->tail_stride_h;
    p.b_tail_len = a->max_tail_len > 0 ? a->b_tail_len : nullptr; p.b_seq_len = a->b_seq_len;
    p.max_tail = a->max_tail_len;
    p.al = a->attn_logits; p.al_sb = a->al_stride_b; p.al_sh = a->al_stride_h; p.al_ss = a->al_stride_s;
    p.S = a->max_seq_len > 0 ? a->num_kv_splits : 0;
    p.o = a->o; p.o_bf16 = (a->o_dtype == OMMX_DT_BF16); p.o_sb = a->o_stride_b; p.o_sh = a->o_stride_h;
    p.lse = a->lse; p.lse_sb = a->lse_stride_b;
    p.sm_scale = a->sm_scale; p.logit_cap = a->logit_cap;
    p.g_world = 0; p.g_rank = 0; p.g_recv = nullptr; p.g_out = nullptr; p.g_state = nullptr; p.status = a->status;
    if (a->gather) {
        const ommx_head_gather *g = a->gather;
        if (g->world < 2 || g->world > 32 || g->rank < 0 || g->rank >= g->world || !g->recv || !g->out || !g->state)
            return fail(OMMX_E_ARG, "head gather: world must be 2..32, rank inside it, and recv / out / state set");
        p.g_world = g->world; p.g_rank = g->rank; p.g_recv = g->recv; p.g_out = g->out; p.g_state = g->state;
    }
    {
        // Stage 1 runs with the largest shared-memory carve-out; asking for the same split here spares the SMs a
        // reconfiguration between the two kernels of every layer.
        static std::atomic<int> carve_set[MAX_DEVICES];
        int dev = 0;
        if (int rc = current_device(&dev)) return rc;
        if (carve_set[dev].load(std::memory_order_acquire) == 0) {
            OMMX_CUDA_TRY(cudaFuncSetAttribute(decode_stage2_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
            carve_set[dev].store(1, std::memory_order_release);
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a->n_q_heads, a->batch);
    cfg.blockDim = dim3(S2_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;   // overlap this kernel's prologue with stage 1's tail
    cfg.attrs = attr;
    cfg.numAttrs = (after_stage1 && a->max_seq_len > 0) ? 1 : 0;
    OMMX_CUDA_TRY(cudaLaunchKernelEx(&cfg, decode_stage2_kernel, p));
    count_launch();
    return 0;
}

}  // namespace ommx

extern "C" int ommx_b200_min_num_kv_splits(int32_t max_seq_len, int32_t page_size) {
    using namespace ommx;
    if (max_seq_len <= 0) return 1;
    int ppg = page_size > 0 && page_size <= 32 ? 32 / page_size : 1;
    int max_groups = MAX_SPLIT_GROUPS;
    if (max_groups * ppg > MAX_SPLIT_PAGES) max_groups = MAX_SPLIT_PAGES / ppg;
    const int groups = (max_seq_len + 31) / 32;
    return (groups + max_groups - 1) / max_groups;
}

extern "C" int ommx_b200_auto_num_kv_splits(int32_t max_seq_len, int32_t batch, int32_t n_kv_heads) {
    (void)n_kv_heads;                       // one CTA serves all local kv heads of its token range
    static std::atomic<int> sm_counts[ommx::MAX_DEVICES];       // per device ordinal
    int dev = 0, sm_count = 148;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < ommx::MAX_DEVICES) {
        sm_count = sm_counts[dev].load(std::memory_order_acquire);
        if (sm_count == 0) {
            int n = 0;
            sm_count = (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 148;
            sm_counts[dev].store(sm_count, std::memory_order_release);
        }
    } else {
        (void)cudaGetLastError();
    }
    // One CTA runs per SM, so a launch takes (waves of CTAs) x (groups per CTA + what a CTA costs before and after its
    // steady state, about three groups' worth).  Pick the split count that minimises it: 148 at batch 1, and e.g. 18
    // rather than 19 at batch 8, where 152 CTAs would leave a second wave of four.  Ties go to fewer splits (less for
    // stage 2 to combine).
    const int groups = max(1, (max_seq_len + 31) / 32);
    const int b = max(1, batch);
    const int s_min = ommx_b200_min_num_kv_splits(max_seq_len, 16);
    const int s_max = max(s_min, min(groups, (4 * sm_count) / b + 1));
    int best = s_min;
    long long best_cost = -1;
    for (int s = s_min; s <= s_max; ++s) {
        const long long waves = ((long long)b * s + sm_count - 1) / sm_count;
        const long long cost = waves * ((groups + s - 1) / s + 3);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s; }
    }
    return max(1, best);
}

extern "C" int ommx_b200_decode_stage1(const ommx_decode_args *a, void *stream) {
    int rc = ommx::validate_decode(a);
    if (rc) return rc;
    return ommx::launch_stage1(a, (cudaStream_t)stream);
}
extern "C" int ommx_b200_decode_stage2(const ommx_decode_args *a, void *stream) {
    int rc = ommx::validate_decode(a);
    if (rc) return rc;
    return ommx::launch_stage2(a, (cudaStream_t)stream);
}
extern "C" int ommx_b200_decode(const ommx_decode_args *a, void *stream) {
    int rc = ommx::validate_decode(a);
    if (rc) return rc;
    rc = ommx::launch_stage1(a, (cudaStream_t)stream);
    if (rc) return rc;
    return ommx::launch_stage2(a, (cudaStream_t)stream, true);
}

// -------------------------------------------------------------------------------------------------
// Decode with the split workspace owned by the library.
//
// Some hosts that embed this library may not allocate device memory at all on their serving path:
// a runtime whose allocator has been frozen after start-up (every later cudaMalloc would fragment or
// overrun a pool sized to the last megabyte), or a plug-in that is handed tensors but no allocator.
// ommx_b200_decode needs a workspace for the per-split partial results; this entry point takes it
// from a fixed array inside the library image instead, so the caller passes only inputs and outputs.
// The array is part of the module: every GPU that loads the library holds its 8 MiB until exit.
constexpr size_t STATIC_WS_FLOATS = (size_t)2 << 20;                      // 2 Mi floats = 8 MiB
static __device__ __align__(256) float g_static_ws[STATIC_WS_FLOATS];

// In host code the name g_static_ws is only a handle, not a device address; the address each
// device gave the array is asked for once per device, with that device current, and kept.
static int static_ws_address(float **out) {
    static std::atomic<float *> cache[64];
    int dev = -1;
    OMMX_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return ommx::fail(OMMX_E_UNSUPPORTED, "decode_static_ws: device ordinal %d", dev);
    float *ptr = cache[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        void *sym = nullptr;
        OMMX_CUDA_TRY(cudaGetSymbolAddress(&sym, g_static_ws));
        if (sym == nullptr) return ommx::fail(OMMX_E_CUDA, "decode_static_ws: the workspace symbol has no address on device %d", dev);
        ptr = static_cast<float *>(sym);
        cache[dev].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return 0;
}

extern "C" int ommx_b200_decode_static_ws(const ommx_decode_args *a, void *stream) {
    using namespace ommx;
    if (!a) return fail(OMMX_E_ARG, "decode_static_ws: null args");
    if (a->batch <= 0 || a->n_q_heads <= 0 || a->num_kv_splits <= 0)
        return fail(OMMX_E_ARG, "decode_static_ws: batch=%d n_q_heads=%d num_kv_splits=%d", a->batch, a->n_q_heads, a->num_kv_splits);
    const size_t row = (size_t)HD + 1;
    const size_t need = (size_t)a->batch * a->n_q_heads * a->num_kv_splits * row;
    if (need > STATIC_WS_FLOATS)
        return fail(OMMX_E_ARG, "decode_static_ws: batch*n_q_heads*num_kv_splits*(head_dim+1) = %zu floats exceeds the "
                                "built-in workspace of %zu floats (8 MiB); use ommx_b200_decode with your own attn_logits",
                    need, (size_t)STATIC_WS_FLOATS);
    float *ws = nullptr;
    int rc = static_ws_address(&ws);
    if (rc) return rc;
    ommx_decode_args b = *a;
    b.attn_logits = ws;
    b.al_stride_s = (int64_t)row;
    b.al_stride_h = (int64_t)a->num_kv_splits * (int64_t)row;
    b.al_stride_b = (int64_t)a->n_q_heads * b.al_stride_h;
    rc = validate_decode(&b);
    if (rc) return rc;
    rc = launch_stage1(&b, (cudaStream_t)stream);
    if (rc) return rc;
    return launch_stage2(&b, (cudaStream_t)stream, true);
}

extern "C" int ommx_b200_merge_states(const float *o_parts, const float *lse_parts, const int32_t *valid_lens,
                                      int32_t P, int32_t R, int32_t D, float *o, float *lse, void *stream) {
    using namespace ommx;
    if (!o_parts || !lse_parts || !o || !lse) return fail(OMMX_E_ARG, "merge: null pointer");
    if (P < 0 || R < 0 || D <= 0) return fail(OMMX_E_ARG, "merge: P=%d R=%d D=%d", P, R, D);
    if (R == 0) return 0;
    merge_states_kernel<<<R, 128, 0, (cudaStream_t)stream>>>(o_parts, lse_parts, valid_lens, P, R, D, o, lse);
    OMMX_CUDA_TRY(cudaGetLastError());
    count_launch();
    return 0;
}
