// Device-resident "lane tile" layout of GGML block-quantized weights.
//
// The bytes a caller uploads are the native GGML rows ([N, bytesPerRow] uint8,
// ml/ggml/dequant.go:31-35 in gomlx/gomlx).  On the device they are kept once, in
// a rearranged order that holds exactly the same bits: the matrix is cut into
// tiles of 16 rows x TK values, and inside a tile the bytes are ordered
// [load j][lane 0..31][16 bytes], so that one warp-wide 128-bit load fetches 512
// contiguous, 16-byte aligned bytes and every lane receives precisely the bytes
// whose values it feeds to the tensor cores.
//
// Lane l = 4*g + t of a warp owns rows g and g+8 of the tile and the K-quarter t
// of the tile (TK/4 consecutive values).  Per format:
//
//   Q4_0  TK=512   j=0: fp16 scales [row g: blocks 4t..4t+3 | row g+8: same]
//                  j=1+2i+r: the 16 nibble bytes of block 4t+i, row g+8r
//   Q8_0  TK=512   j=0: scales as Q4_0
//                  j=1+2(2i+h)+r: int8 values 16h..16h+15 of block 4t+i, row g+8r
//   Q4_K  TK=1024  j=r: the 16 header bytes (d, dmin, scales[12]) of super-block t, row g+8r
//                  j=2+2i+r: bytes 16i..16i+15 of qs[128]
//   Q6_K  TK=1024  j=r: int8 scales[16] of super-block t, row g+8r
//                  j=2+6q+2p+r, q=0..3 (n=q>>1, lh=q&1):
//                      p=0: ql[64n+16lh ..+16]  p=1: ql[64n+32+16lh ..+16]  p=2: qh[32n+16lh ..+16]
//                  then 128 bytes: lane l holds fp16 d of row g, row g+8
//
// Rows beyond N and blocks beyond K are zero-filled (zero scale => zero weight).
#pragma once
#include <cstdint>

namespace b200q {

enum : int { kQ4_0 = 2, kQ8_0 = 8, kQ4_K = 12, kQ6_K = 14, kIQ4_NL = 20 };

template <int TYPE>
struct Fmt;

template <>
struct Fmt<kQ4_0> {
    static constexpr int BPB = 18, VPB = 32, TK = 512, LOADS = 9, TAIL = 0, TILE = LOADS * 512 + TAIL;
    static constexpr int SUB = 32;  // values per aux sub-block (offset term granularity)
    static constexpr bool PERM4 = true;  // x staged as [x0,x2,x1,x3] per group of four
};
template <>
struct Fmt<kQ8_0> {
    static constexpr int BPB = 34, VPB = 32, TK = 512, LOADS = 17, TAIL = 0, TILE = LOADS * 512 + TAIL;
    static constexpr int SUB = 0;
    static constexpr bool PERM4 = false;
};
template <>
struct Fmt<kQ4_K> {
    static constexpr int BPB = 144, VPB = 256, TK = 1024, LOADS = 18, TAIL = 0, TILE = LOADS * 512 + TAIL;
    static constexpr int SUB = 32;
    static constexpr bool PERM4 = true;
};
template <>
struct Fmt<kQ6_K> {
    static constexpr int BPB = 210, VPB = 256, TK = 1024, LOADS = 26, TAIL = 128, TILE = LOADS * 512 + TAIL;
    static constexpr int SUB = 16;
    static constexpr bool PERM4 = false;
};

__host__ __device__ inline int fmt_bpb(int type) {
    return type == kQ4_0 ? 18 : type == kQ8_0 ? 34 : type == kQ4_K ? 144 : type == kQ6_K ? 210 : type == kIQ4_NL ? 18 : 0;
}
__host__ __device__ inline int fmt_vpb(int type) {
    return (type == kQ4_0 || type == kQ8_0 || type == kIQ4_NL) ? 32 : (type == kQ4_K || type == kQ6_K) ? 256 : 0;
}
__host__ __device__ inline int fmt_tk(int type) { return (type == kQ4_0 || type == kQ8_0) ? 512 : 1024; }
__host__ __device__ inline int fmt_tile_bytes(int type) {
    return type == kQ4_0 ? Fmt<kQ4_0>::TILE : type == kQ8_0 ? Fmt<kQ8_0>::TILE : type == kQ4_K ? Fmt<kQ4_K>::TILE
                                                                                                : Fmt<kQ6_K>::TILE;
}

// Byte offset, inside a tile, of byte `o` (0..BPB-1) of block `b` (index inside the
// tile's K range) of tile row `r` (0..15).  This one function defines the layout:
// the upload kernel scatters with it, dequantize / embedding lookup gather with it.
template <int TYPE>
__host__ __device__ inline int tile_byte_offset(int r, int b, int o) {
    const int g = r & 7, rs = r >> 3;
    if constexpr (TYPE == kQ4_0) {
        const int t = b >> 2, i = b & 3, lane = 4 * g + t;
        if (o < 2) return lane * 16 + (rs * 4 + i) * 2 + o;
        return (1 + 2 * i + rs) * 512 + lane * 16 + (o - 2);
    } else if constexpr (TYPE == kQ8_0) {
        const int t = b >> 2, i = b & 3, lane = 4 * g + t;
        if (o < 2) return lane * 16 + (rs * 4 + i) * 2 + o;
        const int q = o - 2, h = q >> 4;
        return (1 + 2 * (2 * i + h) + rs) * 512 + lane * 16 + (q & 15);
    } else if constexpr (TYPE == kQ4_K) {
        const int lane = 4 * g + b;
        if (o < 16) return rs * 512 + lane * 16 + o;
        const int q = o - 16, i = q >> 4;
        return (2 + 2 * i + rs) * 512 + lane * 16 + (q & 15);
    } else {  // Q6_K
        const int lane = 4 * g + b;
        if (o < 128) {  // ql
            const int n = o >> 6, w = o & 63, p = w >> 5, lh = (w >> 4) & 1;
            return (2 + 6 * (2 * n + lh) + 2 * p + rs) * 512 + lane * 16 + (w & 15);
        }
        if (o < 192) {  // qh
            const int w = o - 128, n = w >> 5, lh = (w >> 4) & 1;
            return (2 + 6 * (2 * n + lh) + 4 + rs) * 512 + lane * 16 + (w & 15);
        }
        if (o < 208) return rs * 512 + lane * 16 + (o - 192);  // scales
        return 26 * 512 + lane * 4 + rs * 2 + (o - 208);       // d
    }
}

}  // namespace b200q
