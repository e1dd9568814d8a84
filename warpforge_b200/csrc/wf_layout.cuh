// Device weight layout shared by the repack, dequant-check, GEMV and GEMM kernels.
//
// A weight [rows x K] is cut into tiles of 16 rows x TILE_K columns.  Tiles are stored
// row-tile major, k-tile minor ("stripes" of KT tiles), each tile TILE_BYTES long, the
// whole buffer 256-byte aligned, so a contiguous row range is a contiguous byte range
// (row sharding keeps working) and every 16-byte vector / bulk copy is aligned.
//
// Inside a tile the 4-bit codes are stored in the order the tensor-core A fragment of
// mma.m16n8k16 wants them, so a warp's 32 lanes read 512 contiguous bytes per load and
// never shuffle:
//
//   nibble plane (1024 bytes per 16 rows x 128 k):
//     half h in {0,1} (row = g + 8h), lane t = 4g + q  ->  one uint4 at  h*512 + t*16
//     word j of that uint4 = block j (32 k) of the 128-k group, elements 8q .. 8q+7,
//     element e of those 8 sits at nibble position POS[e] = {0,4,1,5,2,6,3,7}[e], and the
//     whole word is rotated left by 3 bits, so `rotr(w, 4s) & 0x00780078` yields elements
//     (2s, 2s+1) in bits 3..6 of the low / high half -- the top four mantissa bits of a bf16,
//     which OR-ed with an exponent pattern gives (16 + code) without any arithmetic.
//
//   Q4_0  tile = 128 k : plane (codes 0..15, value = code - 8)          1024
//                        fp16 scales [g][row g: blocks 0..3 | row g+8: blocks 0..3]  128
//   Q4_1  tile = 128 k : plane (codes 0..15, value = code * scale + min)  1024
//                        fp16 scales as for Q4_0   128;  fp16 mins, same shape   128
//   Q8_0  tile = 128 k : plane H (high nibble of byte ^ 0x80), plane L (low nibble)  2048
//                        fp16 scales as above                                          128
//   Q5_0  held as Q8_0 tiles (q = code - 16 as the 8-bit integer)
//   Q4_K  tile = 256 k : plane for sub-blocks 0..3, plane for sub-blocks 4..7         2048
//                        (d, dmin) fp16 pairs [g][row g | row g+8]                      64
//                        8-bit sub-block scales [g][row g: 0..7 | row g+8: 0..7]       128
//                        8-bit sub-block mins, same shape                              128
//
// Rows beyond the tensor (rows not a multiple of 16) are stored with zero scales.
#pragma once
#include <stdint.h>

#define WF_QTYPE_Q4_0 2
#define WF_QTYPE_Q4_1 3
#define WF_QTYPE_Q5_0 6
#define WF_QTYPE_Q8_0 8
#define WF_QTYPE_Q4_K 14

#ifdef __CUDACC__
#define WF_HD __host__ __device__ __forceinline__
#else
#define WF_HD inline
#endif

namespace wf {

constexpr int TILE_ROWS = 16;
constexpr int PLANE_BYTES = 1024;  // 16 rows x 128 k of 4-bit codes
constexpr int PLANE_ROT = 3;       // left rotation applied to every plane word

template <int QT> struct Tile;
template <> struct Tile<WF_QTYPE_Q4_0> {
    static constexpr int K = 128, BYTES = 1152, PLANES = 1, BLOCK_K = 32, BLOCK_BYTES = 18;
    static constexpr int SCALE_OFF = 1024;
};
template <> struct Tile<WF_QTYPE_Q4_1> {
    static constexpr int K = 128, BYTES = 1280, PLANES = 1, BLOCK_K = 32, BLOCK_BYTES = 20;
    static constexpr int SCALE_OFF = 1024, MIN_OFF = 1152;
};
template <> struct Tile<WF_QTYPE_Q8_0> {
    static constexpr int K = 128, BYTES = 2176, PLANES = 2, BLOCK_K = 32, BLOCK_BYTES = 34;
    static constexpr int SCALE_OFF = 2048;
};
template <> struct Tile<WF_QTYPE_Q4_K> {
    static constexpr int K = 256, BYTES = 2368, PLANES = 2, BLOCK_K = 256, BLOCK_BYTES = 144;
    static constexpr int D_OFF = 2048, SC_OFF = 2112, MN_OFF = 2240;
};

WF_HD int tile_k(int qt) { return qt == WF_QTYPE_Q4_K ? 256 : 128; }
WF_HD int tile_bytes(int qt) { return qt == WF_QTYPE_Q4_0 ? 1152 : qt == WF_QTYPE_Q4_1 ? 1280 : qt == WF_QTYPE_Q8_0 ? 2176 : 2368; }
WF_HD int block_k(int qt) { return qt == WF_QTYPE_Q4_K ? 256 : 32; }
WF_HD int block_bytes(int qt) { return qt == WF_QTYPE_Q4_0 ? 18 : qt == WF_QTYPE_Q4_1 ? 20 : qt == WF_QTYPE_Q5_0 ? 22 : qt == WF_QTYPE_Q8_0 ? 34 : 144; }
// The format a file type is held in on the device: Q5_0 (value = d * (q5 - 16), an integer in [-16, 15]) is expanded
// into the two 4-bit planes of Q8_0 with the same fp16 scale and runs on the Q8_0 kernels (8 bits per weight in HBM).
WF_HD int device_qtype(int qt) { return qt == WF_QTYPE_Q5_0 ? WF_QTYPE_Q8_0 : qt; }

// Nibble position of element e (0..7) inside its 32-bit word.
WF_HD int nibble_pos(int e) { return (e >> 1) | ((e & 1) << 2); }

// Byte offset inside a plane of the word holding (row r in 0..15, 32-k block j in 0..3,
// element group q in 0..3), and the position of element e = 8q + i.
WF_HD int plane_word_off(int r, int j, int q) { return (r >> 3) * 512 + (((r & 7) << 2) + q) * 16 + j * 4; }

struct WeightGeom {
    int qtype;
    int64_t rows;  // rows in this shard
    int64_t k;     // logical K
    int64_t rt;    // row tiles  = ceil(rows / 16)
    int64_t kt;    // k tiles    = ceil(k / TILE_K)
    int64_t rt_alloc;  // row tiles allocated: rt rounded up to 8, so a 128-row GEMM block never leaves the buffer
    int64_t bytes() const { return rt_alloc * kt * (int64_t)tile_bytes(qtype); }
};

}  // namespace wf
