// Decode GEMV (1 <= m <= 16) for GGML block-quantized weights on sm_100a.
//
// Computes the fused op behind compute.Function.FusedQuantizedDense
// (core/graph/fused_ops.go:195-245 in gomlx/gomlx):
//     y[m, n] = act(sum_k x[m, k] * dequant(W)[n, k] + bias[n])
//
// The kernel is bound by HBM: every packed byte is read exactly once with warp-wide,
// 512-byte contiguous 128-bit loads (see layout.cuh), unpacked in registers, and fed
// straight into m16n8k16 tensor-core MMAs as the A operand (16 weight rows x 16 k),
// with the activations as the B operand (16 k x 8 batch columns) and f32 accumulators.
// Using the tensor cores keeps the instruction count per weight the same for m = 1 and
// m = 16, which is what lets every m in 1..16 run at the memory roofline.
//
// Per-value work:
//   * nibbles / bytes become fp16 through the exponent-magic trick (0x6400 | q is the
//     fp16 number 1024 + q), then one HFMA2 applies the block scale:
//     (1024 + q) * s - 1024 * s = q * s, exact before its single rounding;
//   * the constant offsets of the formats (-8 for Q4_0, -dmin*m for Q4_K, -32 for Q6_K)
//     are not applied per value.  They are linear in the per-sub-block sums of x, so
//     they are added by one extra MMA per tile whose A operand is the per-sub-block
//     coefficient (d, dmin*m, d*sc) and whose B operand is -offset * sum(x) of that
//     sub-block, split into an fp16 high and low part;
//   * Q8_0 is signed and needs no offset: (q + 128 + 1024) - 1152 is exact, then * d.
//
// Activations are rounded to fp16 (saturating at +-65504) when they are staged in
// shared memory; weights are rounded to fp16 after scaling.  Accumulation is f32.
// Relative to the f32 reference this costs about 5e-4 of the output scale.
#include "common.cuh"

#include <algorithm>
#include <cstdlib>

namespace b200q {
namespace {

struct GemvParams {
    const uint8_t *tiles;
    const void *x;
    const float *bias;
    float *y;
    int64_t n, k, y_ld;
    int64_t rt, kt;
    int m, x_dtype, act;
    int ktc;  // k tiles per staged x chunk
};

__device__ __forceinline__ uint4 ldg_stream(const uint8_t *p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
        : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_stream32(const uint8_t *p) {
    uint32_t v;
    asm("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t hfma2u(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hmul2u(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hsub2u(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t bcast_lo(uint32_t p) { return __byte_perm(p, p, 0x1010); }
__device__ __forceinline__ uint32_t bcast_hi(uint32_t p) { return __byte_perm(p, p, 0x3232); }

constexpr uint32_t H2_1024 = 0x64006400u;    // fp16x2 (1024, 1024)
constexpr uint32_t H2_N1024 = 0xE400E400u;   // (-1024, -1024)
constexpr uint32_t H2_N64 = 0xD400D400u;     // (-64, -64)
constexpr uint32_t H2_1152 = 0x64806480u;    // (1152, 1152)
constexpr uint32_t MAGIC_1024 = 0x64006400u; // exponent bits of 1024: low mantissa bits count 1
constexpr uint32_t MAGIC_64 = 0x54005400u;   // exponent bits of 64: mantissa bit 4 counts 1
constexpr uint32_t BYTES_64 = 0x64646464u;

// Two bytes of `v` (selected by `sel`) as the fp16 pair (1024 + b_lo, 1024 + b_hi).
__device__ __forceinline__ uint32_t bytes_to_h2(uint32_t v, uint32_t sel) { return __byte_perm(v, BYTES_64, sel); }
constexpr uint32_t SEL01 = 0x5140, SEL23 = 0x7362;

template <int I>
__device__ __forceinline__ uint32_t word(const uint4 &v) {
    return I == 0 ? v.x : I == 1 ? v.y : I == 2 ? v.z : v.w;
}

// Pointers into the staged activations for the batch columns this lane feeds.
template <int NB>
struct XCols {
    const __half *x[NB];    // row of the staged x chunk
    const __half *shi[NB];  // aux sums, high part
    const __half *slo[NB];  // aux sums, low part
};

// 8 staged activations (16 bytes) of logical chunk `lc` for K-quarter t.  The chunk
// index is XOR-swizzled with 2t when staged, so the four quarters a quad reads in one
// instruction fall into different banks.
__device__ __forceinline__ uint4 lds_chunk(const __half *col, int lc, int t) {
    return *reinterpret_cast<const uint4 *>(col + ((lc ^ (2 * t)) << 3));
}
__device__ __forceinline__ uint2 lds_aux(const __half *s, int idx) {
    return *reinterpret_cast<const uint2 *>(s + idx);
}

// ---------------------------------------------------------------------------------------
// Q4_0 : tile = 16 rows x 512 k, 9 loads per lane.
// ---------------------------------------------------------------------------------------
template <int NB>
__device__ __forceinline__ void tile_q4_0(uint4 (&buf)[9], const uint8_t *nxt, bool has_next, const XCols<NB> &xc,
                                          int lc0, int sub0, float (&acc)[NB][4], int t) {
    const uint4 sc = buf[0];
    if (has_next) buf[0] = ldg_stream(nxt);
#pragma unroll
    for (int nb = 0; nb < NB; nb++) {  // offset term: sum_b d_b * (-8 * sum(x in block b))
        const uint2 bh = lds_aux(xc.shi[nb], sub0 + 4 * t), bl = lds_aux(xc.slo[nb], sub0 + 4 * t);
        mma16816(acc[nb], sc.x, sc.z, sc.y, sc.w, bh.x, bh.y);
        mma16816(acc[nb], sc.x, sc.z, sc.y, sc.w, bl.x, bl.y);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t pg = i < 2 ? sc.x : sc.y, pg8 = i < 2 ? sc.z : sc.w;
        const uint32_t dg = (i & 1) ? bcast_hi(pg) : bcast_lo(pg), dg8 = (i & 1) ? bcast_hi(pg8) : bcast_lo(pg8);
        const uint32_t olo = hmul2u(dg, H2_N1024), ohi = hmul2u(dg, H2_N64);
        const uint32_t olo8 = hmul2u(dg8, H2_N1024), ohi8 = hmul2u(dg8, H2_N64);
        const uint4 qa = buf[1 + 2 * i], qb = buf[2 + 2 * i];
        if (has_next) {
            buf[1 + 2 * i] = ldg_stream(nxt + (1 + 2 * i) * 512);
            buf[2 + 2 * i] = ldg_stream(nxt + (2 + 2 * i) * 512);
        }
        const int lcb = lc0 + 16 * t + 4 * i;
#pragma unroll
        for (int wp = 0; wp < 2; wp++) {
            uint4 blo[NB], bhi[NB];
#pragma unroll
            for (int nb = 0; nb < NB; nb++) {
                blo[nb] = lds_chunk(xc.x[nb], lcb + wp, t);
                bhi[nb] = lds_chunk(xc.x[nb], lcb + 2 + wp, t);
            }
#pragma unroll
            for (int ww = 0; ww < 2; ww++) {
                const uint32_t wa = wp == 0 ? (ww == 0 ? qa.x : qa.y) : (ww == 0 ? qa.z : qa.w);
                const uint32_t wb = wp == 0 ? (ww == 0 ? qb.x : qb.y) : (ww == 0 ? qb.z : qb.w);
                const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
                const uint32_t l0 = hfma2u((wa & 0x000F000Fu) | MAGIC_1024, dg, olo);
                const uint32_t l1 = hfma2u((wb & 0x000F000Fu) | MAGIC_1024, dg8, olo8);
                const uint32_t l2 = hfma2u((wa8 & 0x000F000Fu) | MAGIC_1024, dg, olo);
                const uint32_t l3 = hfma2u((wb8 & 0x000F000Fu) | MAGIC_1024, dg8, olo8);
                const uint32_t h0 = hfma2u((wa & 0x00F000F0u) | MAGIC_64, dg, ohi);
                const uint32_t h1 = hfma2u((wb & 0x00F000F0u) | MAGIC_64, dg8, ohi8);
                const uint32_t h2 = hfma2u((wa8 & 0x00F000F0u) | MAGIC_64, dg, ohi);
                const uint32_t h3 = hfma2u((wb8 & 0x00F000F0u) | MAGIC_64, dg8, ohi8);
#pragma unroll
                for (int nb = 0; nb < NB; nb++) {
                    mma16816(acc[nb], l0, l1, l2, l3, ww == 0 ? blo[nb].x : blo[nb].z, ww == 0 ? blo[nb].y : blo[nb].w);
                    mma16816(acc[nb], h0, h1, h2, h3, ww == 0 ? bhi[nb].x : bhi[nb].z, ww == 0 ? bhi[nb].y : bhi[nb].w);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Q8_0 : tile = 16 rows x 512 k, 17 loads per lane.
// ---------------------------------------------------------------------------------------
template <int NB>
__device__ __forceinline__ void tile_q8_0(uint4 (&buf)[17], const uint8_t *nxt, bool has_next, const XCols<NB> &xc,
                                          int lc0, float (&acc)[NB][4], int t) {
    const uint4 sc = buf[0];
    if (has_next) buf[0] = ldg_stream(nxt);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t pg = i < 2 ? sc.x : sc.y, pg8 = i < 2 ? sc.z : sc.w;
        const uint32_t dg = (i & 1) ? bcast_hi(pg) : bcast_lo(pg), dg8 = (i & 1) ? bcast_hi(pg8) : bcast_lo(pg8);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int j = 1 + 2 * (2 * i + h);
            const uint4 qa = buf[j], qb = buf[j + 1];
            if (has_next) {
                buf[j] = ldg_stream(nxt + j * 512);
                buf[j + 1] = ldg_stream(nxt + (j + 1) * 512);
            }
            const int lcb = lc0 + 16 * t + 4 * i + 2 * h;
#pragma unroll
            for (int wp = 0; wp < 2; wp++) {
                uint4 b[NB];
#pragma unroll
                for (int nb = 0; nb < NB; nb++) b[nb] = lds_chunk(xc.x[nb], lcb + wp, t);
#pragma unroll
                for (int ww = 0; ww < 2; ww++) {
                    const uint32_t wa = (wp == 0 ? (ww == 0 ? qa.x : qa.y) : (ww == 0 ? qa.z : qa.w)) ^ 0x80808080u;
                    const uint32_t wb = (wp == 0 ? (ww == 0 ? qb.x : qb.y) : (ww == 0 ? qb.z : qb.w)) ^ 0x80808080u;
                    const uint32_t a0 = hmul2u(hsub2u(bytes_to_h2(wa, SEL01), H2_1152), dg);
                    const uint32_t a1 = hmul2u(hsub2u(bytes_to_h2(wb, SEL01), H2_1152), dg8);
                    const uint32_t a2 = hmul2u(hsub2u(bytes_to_h2(wa, SEL23), H2_1152), dg);
                    const uint32_t a3 = hmul2u(hsub2u(bytes_to_h2(wb, SEL23), H2_1152), dg8);
#pragma unroll
                    for (int nb = 0; nb < NB; nb++)
                        mma16816(acc[nb], a0, a1, a2, a3, ww == 0 ? b[nb].x : b[nb].z, ww == 0 ? b[nb].y : b[nb].w);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Q4_K : tile = 16 rows x 1024 k (4 super-blocks, one per quad lane), 18 loads per lane.
// ---------------------------------------------------------------------------------------
// Header (d, dmin, scales[12]) -> fp16 pairs ds[j/2] = d*sc_j and cm[j/2] = dmin*m_j.
__device__ __forceinline__ void q4k_header(const uint4 &h, uint32_t (&ds)[4], uint32_t (&cm)[4]) {
    const uint32_t d2 = bcast_lo(h.x), dmin2 = bcast_hi(h.x);
    const uint32_t sc0 = h.y & 0x3F3F3F3Fu, m0 = h.z & 0x3F3F3F3Fu;
    const uint32_t sc1 = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
    const uint32_t m1 = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
    ds[0] = hmul2u(hsub2u(bytes_to_h2(sc0, SEL01), H2_1024), d2);
    ds[1] = hmul2u(hsub2u(bytes_to_h2(sc0, SEL23), H2_1024), d2);
    ds[2] = hmul2u(hsub2u(bytes_to_h2(sc1, SEL01), H2_1024), d2);
    ds[3] = hmul2u(hsub2u(bytes_to_h2(sc1, SEL23), H2_1024), d2);
    cm[0] = hmul2u(hsub2u(bytes_to_h2(m0, SEL01), H2_1024), dmin2);
    cm[1] = hmul2u(hsub2u(bytes_to_h2(m0, SEL23), H2_1024), dmin2);
    cm[2] = hmul2u(hsub2u(bytes_to_h2(m1, SEL01), H2_1024), dmin2);
    cm[3] = hmul2u(hsub2u(bytes_to_h2(m1, SEL23), H2_1024), dmin2);
}

template <int NB>
__device__ __forceinline__ void tile_q4_k(uint4 (&buf)[18], const uint8_t *nxt, bool has_next, const XCols<NB> &xc,
                                          int lc0, int sub0, float (&acc)[NB][4], int t) {
    uint32_t dsA[4], cmA[4], dsB[4], cmB[4];
    q4k_header(buf[0], dsA, cmA);
    q4k_header(buf[1], dsB, cmB);
    if (has_next) {
        buf[0] = ldg_stream(nxt);
        buf[1] = ldg_stream(nxt + 512);
    }
#pragma unroll
    for (int nb = 0; nb < NB; nb++) {  // offset term: sum_j (dmin*m_j) * (-sum(x in sub-block j))
#pragma unroll
        for (int q = 0; q < 2; q++) {
            const uint2 bh = lds_aux(xc.shi[nb], sub0 + 8 * t + 4 * q), bl = lds_aux(xc.slo[nb], sub0 + 8 * t + 4 * q);
            mma16816(acc[nb], cmA[2 * q], cmB[2 * q], cmA[2 * q + 1], cmB[2 * q + 1], bh.x, bh.y);
            mma16816(acc[nb], cmA[2 * q], cmB[2 * q], cmA[2 * q + 1], cmB[2 * q + 1], bl.x, bl.y);
        }
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int G = i >> 1, hf = i & 1;
        // low nibbles: sub-block 2G (low half of pair G); high nibbles: sub-block 2G+1.
        const uint32_t sl = bcast_lo(dsA[G]), sh = bcast_hi(dsA[G]), sl8 = bcast_lo(dsB[G]), sh8 = bcast_hi(dsB[G]);
        const uint32_t olo = hmul2u(sl, H2_N1024), ohi = hmul2u(sh, H2_N64);
        const uint32_t olo8 = hmul2u(sl8, H2_N1024), ohi8 = hmul2u(sh8, H2_N64);
        const uint4 qa = buf[2 + 2 * i], qb = buf[3 + 2 * i];
        if (has_next) {
            buf[2 + 2 * i] = ldg_stream(nxt + (2 + 2 * i) * 512);
            buf[3 + 2 * i] = ldg_stream(nxt + (3 + 2 * i) * 512);
        }
        const int lcb = lc0 + 32 * t + 8 * G + 2 * hf;
#pragma unroll
        for (int wp = 0; wp < 2; wp++) {
            uint4 blo[NB], bhi[NB];
#pragma unroll
            for (int nb = 0; nb < NB; nb++) {
                blo[nb] = lds_chunk(xc.x[nb], lcb + wp, t);
                bhi[nb] = lds_chunk(xc.x[nb], lcb + 4 + wp, t);
            }
#pragma unroll
            for (int ww = 0; ww < 2; ww++) {
                const uint32_t wa = wp == 0 ? (ww == 0 ? qa.x : qa.y) : (ww == 0 ? qa.z : qa.w);
                const uint32_t wb = wp == 0 ? (ww == 0 ? qb.x : qb.y) : (ww == 0 ? qb.z : qb.w);
                const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
                const uint32_t l0 = hfma2u((wa & 0x000F000Fu) | MAGIC_1024, sl, olo);
                const uint32_t l1 = hfma2u((wb & 0x000F000Fu) | MAGIC_1024, sl8, olo8);
                const uint32_t l2 = hfma2u((wa8 & 0x000F000Fu) | MAGIC_1024, sl, olo);
                const uint32_t l3 = hfma2u((wb8 & 0x000F000Fu) | MAGIC_1024, sl8, olo8);
                const uint32_t h0 = hfma2u((wa & 0x00F000F0u) | MAGIC_64, sh, ohi);
                const uint32_t h1 = hfma2u((wb & 0x00F000F0u) | MAGIC_64, sh8, ohi8);
                const uint32_t h2 = hfma2u((wa8 & 0x00F000F0u) | MAGIC_64, sh, ohi);
                const uint32_t h3 = hfma2u((wb8 & 0x00F000F0u) | MAGIC_64, sh8, ohi8);
#pragma unroll
                for (int nb = 0; nb < NB; nb++) {
                    mma16816(acc[nb], l0, l1, l2, l3, ww == 0 ? blo[nb].x : blo[nb].z, ww == 0 ? blo[nb].y : blo[nb].w);
                    mma16816(acc[nb], h0, h1, h2, h3, ww == 0 ? bhi[nb].x : bhi[nb].z, ww == 0 ? bhi[nb].y : bhi[nb].w);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Q6_K : tile = 16 rows x 1024 k (4 super-blocks), 26 loads + one 4-byte load per lane.
// ---------------------------------------------------------------------------------------
// int8 scales[16] and d -> fp16 pairs ds[s/2] = d * sc_s.
__device__ __forceinline__ void q6k_scales(const uint4 &s, uint32_t d2, uint32_t (&ds)[8]) {
    const uint32_t w[4] = {s.x ^ 0x80808080u, s.y ^ 0x80808080u, s.z ^ 0x80808080u, s.w ^ 0x80808080u};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        ds[2 * i] = hmul2u(hsub2u(bytes_to_h2(w[i], SEL01), H2_1152), d2);
        ds[2 * i + 1] = hmul2u(hsub2u(bytes_to_h2(w[i], SEL23), H2_1152), d2);
    }
}

template <int NB>
__device__ __forceinline__ void tile_q6_k(uint4 (&buf)[26], uint32_t &tail, const uint8_t *nxt, const uint8_t *nxt_tail,
                                          bool has_next, const XCols<NB> &xc, int lc0, int sub0, float (&acc)[NB][4],
                                          int t) {
    uint32_t dsA[8], dsB[8];
    q6k_scales(buf[0], bcast_lo(tail), dsA);
    q6k_scales(buf[1], bcast_hi(tail), dsB);
    if (has_next) {
        buf[0] = ldg_stream(nxt);
        buf[1] = ldg_stream(nxt + 512);
        tail = ldg_stream32(nxt_tail);
    }
#pragma unroll
    for (int nb = 0; nb < NB; nb++) {  // offset term: sum_s (d*sc_s) * (-32 * sum(x in sub-block s))
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const uint2 bh = lds_aux(xc.shi[nb], sub0 + 16 * t + 4 * q), bl = lds_aux(xc.slo[nb], sub0 + 16 * t + 4 * q);
            mma16816(acc[nb], dsA[2 * q], dsB[2 * q], dsA[2 * q + 1], dsB[2 * q + 1], bh.x, bh.y);
            mma16816(acc[nb], dsA[2 * q], dsB[2 * q], dsA[2 * q + 1], dsB[2 * q + 1], bl.x, bl.y);
        }
    }
#pragma unroll
    for (int gr = 0; gr < 4; gr++) {
        const int n = gr >> 1, lh = gr & 1, j0 = 2 + 6 * gr;
        const uint4 la = buf[j0], la8 = buf[j0 + 1], lb = buf[j0 + 2], lb8 = buf[j0 + 3], hh = buf[j0 + 4],
                    hh8 = buf[j0 + 5];
        if (has_next) {
#pragma unroll
            for (int u = 0; u < 6; u++) buf[j0 + u] = ldg_stream(nxt + (j0 + u) * 512);
        }
        uint32_t s[4], s8[4], o[4], o8[4];
#pragma unroll
        for (int c = 0; c < 4; c++) {  // code c uses scale 8n + lh + 2c = half lh of pair 4n + c
            s[c] = lh ? bcast_hi(dsA[4 * n + c]) : bcast_lo(dsA[4 * n + c]);
            s8[c] = lh ? bcast_hi(dsB[4 * n + c]) : bcast_lo(dsB[4 * n + c]);
            o[c] = hmul2u(s[c], H2_N1024);
            o8[c] = hmul2u(s8[c], H2_N1024);
        }
        const int lcb = lc0 + 32 * t + 16 * n + 2 * lh;
#pragma unroll
        for (int wp = 0; wp < 2; wp++) {
            uint4 b[4][NB];
#pragma unroll
            for (int c = 0; c < 4; c++)
#pragma unroll
                for (int nb = 0; nb < NB; nb++) b[c][nb] = lds_chunk(xc.x[nb], lcb + 4 * c + wp, t);
#pragma unroll
            for (int ww = 0; ww < 2; ww++) {
                const uint32_t a = wp == 0 ? (ww == 0 ? la.x : la.y) : (ww == 0 ? la.z : la.w);
                const uint32_t a8 = wp == 0 ? (ww == 0 ? la8.x : la8.y) : (ww == 0 ? la8.z : la8.w);
                const uint32_t bq = wp == 0 ? (ww == 0 ? lb.x : lb.y) : (ww == 0 ? lb.z : lb.w);
                const uint32_t bq8 = wp == 0 ? (ww == 0 ? lb8.x : lb8.y) : (ww == 0 ? lb8.z : lb8.w);
                const uint32_t h = wp == 0 ? (ww == 0 ? hh.x : hh.y) : (ww == 0 ? hh.z : hh.w);
                const uint32_t h8 = wp == 0 ? (ww == 0 ? hh8.x : hh8.y) : (ww == 0 ? hh8.z : hh8.w);
                uint32_t code[4], code8[4];
                code[0] = (a & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u);
                code[1] = (bq & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u);
                code[2] = ((a >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u);
                code[3] = ((bq >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u);
                code8[0] = (a8 & 0x0F0F0F0Fu) | ((h8 << 4) & 0x30303030u);
                code8[1] = (bq8 & 0x0F0F0F0Fu) | ((h8 << 2) & 0x30303030u);
                code8[2] = ((a8 >> 4) & 0x0F0F0F0Fu) | (h8 & 0x30303030u);
                code8[3] = ((bq8 >> 4) & 0x0F0F0F0Fu) | ((h8 >> 2) & 0x30303030u);
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const uint32_t a0 = hfma2u(bytes_to_h2(code[c], SEL01), s[c], o[c]);
                    const uint32_t a1 = hfma2u(bytes_to_h2(code8[c], SEL01), s8[c], o8[c]);
                    const uint32_t a2 = hfma2u(bytes_to_h2(code[c], SEL23), s[c], o[c]);
                    const uint32_t a3 = hfma2u(bytes_to_h2(code8[c], SEL23), s8[c], o8[c]);
#pragma unroll
                    for (int nb = 0; nb < NB; nb++)
                        mma16816(acc[nb], a0, a1, a2, a3, ww == 0 ? b[c][nb].x : b[c][nb].z,
                                 ww == 0 ? b[c][nb].y : b[c][nb].w);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Activation staging: x[m, k0 .. k0+kc) -> fp16 in shared memory, plus the per-sub-block
// sums needed by the offset MMAs.  One thread handles 8 consecutive values.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t f2h2_sat(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

template <int TYPE>
__device__ __forceinline__ void stage_x(const GemvParams &p, int64_t k0, int kc, int xs_stride, int ns, __half *xs,
                                        __half *shi, __half *slo) {
    using F = Fmt<TYPE>;
    const int gpc = kc >> 3;  // 8-value groups per column, a multiple of 64
    const int total = p.m * gpc;
    for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
        const int col = idx / gpc, gi = idx - col * gpc;
        const int64_t k = k0 + (int64_t)gi * 8;
        float v[8];
        if (k < p.k) {
            if (p.x_dtype == B200Q_F32) {
                const float4 *src = reinterpret_cast<const float4 *>(static_cast<const float *>(p.x) + col * p.k + k);
                const float4 a = __ldg(src), b = __ldg(src + 1);
                v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
            } else {
                const uint4 r =
                    __ldg(reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(p.x) + col * p.k + k));
                const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    v[2 * i] = __uint_as_float(w[i] << 16);
                    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = 0.0f;
        }
        uint4 out;
        if constexpr (F::PERM4) {
            out.x = f2h2_sat(v[0], v[2]), out.y = f2h2_sat(v[1], v[3]);
            out.z = f2h2_sat(v[4], v[6]), out.w = f2h2_sat(v[5], v[7]);
        } else {
            out.x = f2h2_sat(v[0], v[1]), out.y = f2h2_sat(v[2], v[3]);
            out.z = f2h2_sat(v[4], v[5]), out.w = f2h2_sat(v[6], v[7]);
        }
        const int tq = ((gi << 3) & (F::TK - 1)) / (F::TK / 4);
        *reinterpret_cast<uint4 *>(xs + col * xs_stride + ((gi ^ (2 * tq)) << 3)) = out;
        if constexpr (F::SUB != 0) {
            // Sums are taken over the rounded values the MMAs will see, so the offset cancels exactly.
            const uint32_t w[4] = {out.x, out.y, out.z, out.w};
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
                sum += f.x + f.y;
            }
            constexpr float OFFSET = TYPE == kQ4_0 ? 8.0f : TYPE == kQ4_K ? 1.0f : 32.0f;
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            if constexpr (F::SUB == 32) sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            constexpr int GPS = F::SUB / 8;  // groups per sub-block
            if ((gi & (GPS - 1)) == 0) {
                const float s = -OFFSET * sum;
                const __half hi = __float2half_rn(s);
                const __half lo = __float2half_rn(s - __half2float(hi));
                shi[col * ns + gi / GPS] = hi;
                slo[col * ns + gi / GPS] = lo;
            }
        }
    }
}

template <int TYPE, int NB>
__global__ void __launch_bounds__(256) gemv_mma_kernel(const GemvParams p) {
    using F = Fmt<TYPE>;
    extern __shared__ __align__(16) uint8_t smem[];
    const int kc_max = p.ktc * F::TK;
    const int xs_stride = kc_max + 8;
    const int ns = F::SUB ? kc_max / F::SUB : 0;
    __half *xs = reinterpret_cast<__half *>(smem);
    __half *shi = xs + (size_t)p.m * xs_stride;
    __half *slo = shi + (size_t)p.m * ns;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int64_t rt = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
    const bool active = rt < p.rt;
    const uint8_t *wbase = p.tiles + (active ? rt : 0) * p.kt * (int64_t)F::TILE + lane * 16;
    const uint8_t *tbase = p.tiles + (active ? rt : 0) * p.kt * (int64_t)F::TILE + F::LOADS * 512 + lane * 4;

    uint4 buf[F::LOADS];
    uint32_t tail = 0;
    if (active) {
#pragma unroll
        for (int j = 0; j < F::LOADS; j++) buf[j] = ldg_stream(wbase + j * 512);
        if constexpr (F::TAIL != 0) tail = ldg_stream32(tbase);
    }

    XCols<NB> xc;
#pragma unroll
    for (int nb = 0; nb < NB; nb++) {
        const int col = min(g + 8 * nb, p.m - 1);
        xc.x[nb] = xs + col * xs_stride;
        xc.shi[nb] = shi + col * ns;
        xc.slo[nb] = slo + col * ns;
    }

    float acc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; nb++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[nb][i] = 0.0f;

    for (int64_t kt0 = 0; kt0 < p.kt; kt0 += p.ktc) {
        const int nkt = (int)min((int64_t)p.ktc, p.kt - kt0);
        if (kt0 != 0) __syncthreads();  // everyone is done reading the previous chunk
        stage_x<TYPE>(p, kt0 * F::TK, nkt * F::TK, xs_stride, ns, xs, shi, slo);
        __syncthreads();
        if (active) {
            for (int kl = 0; kl < nkt; kl++) {
                const int64_t kt = kt0 + kl;
                const bool has_next = kt + 1 < p.kt;
                const uint8_t *nxt = wbase + (kt + 1) * (int64_t)F::TILE;
                const int lc0 = kl * (F::TK / 8);
                if constexpr (TYPE == kQ4_0) {
                    tile_q4_0<NB>(buf, nxt, has_next, xc, lc0, kl * (F::TK / 32), acc, t);
                } else if constexpr (TYPE == kQ8_0) {
                    tile_q8_0<NB>(buf, nxt, has_next, xc, lc0, acc, t);
                } else if constexpr (TYPE == kQ4_K) {
                    tile_q4_k<NB>(buf, nxt, has_next, xc, lc0, kl * (F::TK / 32), acc, t);
                } else {
                    tile_q6_k<NB>(buf, tail, nxt, tbase + (kt + 1) * (int64_t)F::TILE, has_next, xc, lc0,
                                  kl * (F::TK / 16), acc, t);
                }
            }
        }
    }

    if (active) {
        // D fragment: rows g, g+8 of the tile; batch columns 2t, 2t+1 (+8 per nb).
#pragma unroll
        for (int nb = 0; nb < NB; nb++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int64_t row = rt * 16 + g + 8 * (i >> 1);
                const int col = 8 * nb + 2 * t + (i & 1);
                if (row < p.n && col < p.m) {
                    float v = acc[nb][i];
                    if (p.bias != nullptr) v += __ldg(p.bias + row);
                    p.y[(int64_t)col * p.y_ld + row] = apply_activation(p.act, v);
                }
            }
    }
}

int env_int(const char *name, int dflt) {
    const char *v = std::getenv(name);
    return v && *v ? std::atoi(v) : dflt;
}

template <int TYPE, int NB>
int launch_t(const Weight &w, const GemvParams &p0, cudaStream_t s) {
    using F = Fmt<TYPE>;
    GemvParams p = p0;
    // Warps per CTA: more rows per CTA amortise the activation staging when m is large.
    int warps = env_int("B200Q_GEMV_WARPS", p.m > 4 ? 8 : 4);
    warps = std::max(1, std::min(8, warps));
    // Largest staged chunk that keeps shared memory within the budget.
    const int smem_budget = env_int("B200Q_GEMV_SMEM", 72 * 1024);
    const int per_tile = p.m * (F::TK * 2 + (F::SUB ? 2 * 2 * (F::TK / F::SUB) : 0));
    int ktc = (smem_budget - p.m * 16) / per_tile;
    ktc = (int)std::max<int64_t>(1, std::min<int64_t>(ktc, w.kt));
    p.ktc = ktc;
    const size_t smem = (size_t)p.m * (ktc * F::TK + 8) * 2 + (F::SUB ? (size_t)p.m * (ktc * F::TK / F::SUB) * 4 : 0);
    auto kern = gemv_mma_kernel<TYPE, NB>;
    static thread_local size_t configured[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (smem > configured[w.device & 7]) {
        B200Q_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured[w.device & 7] = 200 * 1024;
    }
    const int64_t grid = (w.rt + warps - 1) / warps;
    kern<<<(unsigned)grid, warps * 32, smem, s>>>(p);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : cuda_fail(e, "gemv launch");
}

template <int TYPE>
int launch_nb(const Weight &w, const GemvParams &p, cudaStream_t s) {
    return p.m <= 8 ? launch_t<TYPE, 1>(w, p, s) : launch_t<TYPE, 2>(w, p, s);
}

}  // namespace

int launch_gemv(const Weight &w, const void *x, int x_dtype, int m, const float *bias, int act, float *y, int64_t y_ld,
                cudaStream_t s) {
    if (m < 1 || m > 16) return fail(B200Q_EINVAL, "gemv: m must be in 1..16");
    GemvParams p{};
    p.tiles = w.tiles;
    p.x = x;
    p.bias = bias;
    p.y = y;
    p.n = w.n, p.k = w.k, p.y_ld = y_ld;
    p.rt = w.rt, p.kt = w.kt;
    p.m = m, p.x_dtype = x_dtype, p.act = act;
    switch (w.type) {
    case kQ4_0: return launch_nb<kQ4_0>(w, p, s);
    case kQ8_0: return launch_nb<kQ8_0>(w, p, s);
    case kQ4_K: return launch_nb<kQ4_K>(w, p, s);
    case kQ6_K: return launch_nb<kQ6_K>(w, p, s);
    }
    return fail(B200Q_ENOTIMPL, "gemv: unsupported GGML type");
}

}  // namespace b200q
