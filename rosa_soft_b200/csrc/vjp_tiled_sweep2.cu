// Second sweep of the dense surrogate VJP, register-tiled: the same schedule and tensor-core
// contraction as vjp_sweep2_tc_kernel (surrogate_vjp.cu) with TWO consecutive diagonals per
// thread and 128 threads per band of 256 diagonals.
//
// Per row block (16 rows, bottom-up): the forward recurrence is re-run from the block's
// checkpoint (evidence S kept in a thread-private shared-memory column, the mismatch counts
// packed into bytes), the adjoint recurrence runs backwards over it and writes the cell adjoint
// C and the weighted probability p*d as bf16 terms into one un-skewed [row][window column]
// operand area, and tcgen05.mma contracts that area three ways (column sums C^T qz and
// (p d)^T gO, row sums C kz) into fp32 accumulators in tensor memory.  The MMAs of block b run
// while the tables and the forward phase of block b+1 are computed; their accumulators are
// added to the CTA-owned partial gradient rows (vector reductions to L2, first touch a store)
// just before block b+1 overwrites the operands.  The kernel text lives in
// vjp_tiled_sweep2_kernel.inl and is expanded twice: one block per flush of the column sums for
// value rows of up to 16 components, two blocks per flush for wider rows.
//
// What the two-diagonal tiling buys: key-side tables of four rows are six consecutive columns
// held in registers (64-bit shared loads), row-only values are loaded once for two cells, on
// even rows the two cells of a thread are one aligned 32-bit operand store per term, S and the
// packed mismatch counts move as 64-bit words, and blocks whose cells are all active and past
// the horizon run without per-cell predicates.
//
// Operand precision follows the input dtype: float32 inputs keep three bf16 terms of C (24
// mantissa bits, the row sums cancel heavily) and two of p*d; float16 inputs two and two;
// bfloat16 inputs two terms of C and one of p*d -- their gradients are compared at the half
// precision tolerances of the operator contract (3e-3 / 2e-2), far above what is dropped.
#include "common.cuh"
#include "tcgen05.cuh"
#include "vjp_shared.cuh"
#include "vjp_tiled.cuh"

namespace rosa {

namespace {

constexpr int kS2Threads = 128;
constexpr int kS2R = 2;                              // diagonals per thread
constexpr int kS2Band = kVjpBand;                    // 256 diagonals per band
constexpr int kS2Rows = kVjpRows;                    // 16
constexpr int kS2Win = kS2Band + kS2Rows;            // 272 window columns of one block
// Value rows wider than 16 components (the epilogue then moves three times the data): the column
// sums of TWO consecutive blocks of a band are accumulated in tensor memory before they are added
// to the partial rows.  The window of the second block lies 16 columns lower, so the operand area
// spans 288 columns, the first block of a pair writes its cells 16 columns up, the second at
// column 0, and tile column t of either is key position (window base of the second block) + t.
// Narrow value rows keep one block per flush and a 272-column area: pairing measured slower
// there (169.5 against 158.7 ms at the headline shape; 39.5 against 44.6 ms on the packed
// fp16 workload with 32 value components).
__host__ __device__ constexpr bool pairs_blocks(int NV) { return NV > 16; }
__host__ __device__ constexpr int tile_cols(int NV) {
  return pairs_blocks(NV) ? kS2Win + kS2Rows : kS2Win;
}
constexpr int kS2NK = 16;                            // symbol bits padded to one MMA N
static_assert(kS2Threads * kS2R == kS2Band && kS2Rows == 16, "tile geometry");

// Operand area: core matrices of 8 rows x 16 bytes, ordered [column group][term][row group],
// 144 bytes apart inside a term (128 + 16 of skew), terms 288 bytes apart, column groups
// NT * 288 + 16 bytes apart (an odd multiple of 16, so that the 32-bit stores of a warp -- 8
// column groups, 4 lanes per 16-byte core row -- fall into 32 different banks).
constexpr int kRowGroupBytes = 144;
constexpr int kTermBytes = 2 * kRowGroupBytes;
__host__ __device__ constexpr int col_group_bytes(int nterms) { return nterms * kTermBytes + 16; }
__host__ __device__ constexpr int operand_bytes(int nterms, int cols = kS2Win) {
  // the K-major view with M = 64 reads eight cores (1152 bytes) from every column group start:
  // keep that much readable after the last group
  return (cols / 8) * col_group_bytes(nterms) + 8 * kRowGroupBytes;
}
__host__ __device__ constexpr int chunk_start(int ch, int cols = kS2Win) {
  return ch == 0 ? 0 : ch == 1 ? 128 : cols - 128;
}
// B operand tiles, K-major: element (n, k) of an N x K matrix
__device__ __forceinline__ int b_off(int n, int k, int N) {
  return (k >> 3) * (N / 8 * 128) + (n >> 3) * 128 + (n & 7) * 16 + (k & 7) * 2;
}

// precision policy per input dtype
template <int kPrec> struct Terms;               // 0 float32, 1 float16, 2 bfloat16
template <> struct Terms<0> { static constexpr int C = 3, P = 2; static constexpr bool glo = true; };
template <> struct Terms<1> { static constexpr int C = 2, P = 2; static constexpr bool glo = true; };
template <> struct Terms<2> { static constexpr int C = 2, P = 1; static constexpr bool glo = false; };

__device__ __forceinline__ uint32_t hi_bits(float v) { return __float_as_uint(v) & 0xffff0000u; }
// (upper half of b) << 16 | upper half of a
__device__ __forceinline__ uint32_t pack_hi(uint32_t a, uint32_t b) {
  return __byte_perm(a, b, 0x7632);
}
__device__ __forceinline__ uint32_t pack_rn(float a, float b) {   // bf16(b) << 16 | bf16(a)
  const __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&p);
}

// Splits two neighbouring cells (column c: lo half, column c + 1: hi half) into NT bf16 terms.
// kRound = false: the leading terms by truncation (one mask each; their remainder is exact in
// float32), the last by rounding.  kRound = true (float32 inputs): every term rounded to nearest,
// which halves the representation error of the last term.
template <int NT, bool kRound>
__device__ __forceinline__ void split_pair(float a, float b, uint32_t (&out)[3]) {
  if (NT == 1) {
    out[0] = pack_rn(a, b);
    return;
  }
  float ra, rb;
  if (kRound) {
    out[0] = pack_rn(a, b);
    ra = a - __uint_as_float(out[0] << 16);
    rb = b - __uint_as_float(out[0] & 0xffff0000u);
  } else {
    const uint32_t a0 = hi_bits(a), b0 = hi_bits(b);
    out[0] = pack_hi(a0, b0);
    ra = a - __uint_as_float(a0);
    rb = b - __uint_as_float(b0);
  }
  if (NT == 2) {
    out[1] = pack_rn(ra, rb);
    return;
  }
  float sa, sb2;
  if (kRound) {
    out[1] = pack_rn(ra, rb);
    sa = ra - __uint_as_float(out[1] << 16);
    sb2 = rb - __uint_as_float(out[1] & 0xffff0000u);
  } else {
    const uint32_t a1 = hi_bits(ra), b1 = hi_bits(rb);
    out[1] = pack_hi(a1, b1);
    sa = ra - __uint_as_float(a1);
    sb2 = rb - __uint_as_float(b1);
  }
  out[2] = pack_rn(sa, sb2);
}

// Stores the terms of two cells: `aligned` (even column first) as one 32-bit word per term at
// byte offset `off_lo`; otherwise the low cell at `off_lo` and the high cell at `off_hi` as
// 16-bit halves.
template <int NT, bool kRound>
__device__ __forceinline__ void store_pair(unsigned char* term0, int off_lo, int off_hi,
                                           bool aligned, float lo_cell, float hi_cell) {
  uint32_t w[3];
  split_pair<NT, kRound>(lo_cell, hi_cell, w);
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    unsigned char* base = term0 + t * kTermBytes;
    if (aligned) {
      *reinterpret_cast<uint32_t*>(base + off_lo) = w[t];
    } else {
      *reinterpret_cast<uint16_t*>(base + off_lo) = (uint16_t)(w[t] & 0xffffu);
      *reinterpret_cast<uint16_t*>(base + off_hi) = (uint16_t)(w[t] >> 16);
    }
  }
}

// byte offset of window column c inside a term row (row part added by the caller)
__device__ __forceinline__ int col_off(int c, int cg_bytes) {
  return (c >> 3) * cg_bytes + (c & 7) * 2;
}
__device__ __forceinline__ int row_off(int r) { return (r >> 3) * kRowGroupBytes + (r & 7) * 16; }

// Shared-memory plan (bytes from the start of dynamic shared memory).
template <int NV, int NG, int kPrec>
struct S2Smem {
  static constexpr int kTerms = Terms<kPrec>::C + Terms<kPrec>::P;
  static constexpr int kCg = col_group_bytes(kTerms);
  static constexpr int kKzSlots = kS2Win / 16 + 2;              // circular k-steps of kz^T
  static constexpr int kKzSlotBytes = kS2NK * 32;               // [NK][16] bf16
  static constexpr int kQzBytes = kS2NK * kS2Rows * 2;
  static constexpr int kGBytes = NV * kS2Rows * 2;
  static constexpr int oTile = 0;
  static constexpr int kTileCols = tile_cols(NV);
  static constexpr int oQz = operand_bytes(kTerms, kTileCols);  // two buffers
  static constexpr int oGhi = oQz + 2 * kQzBytes;               // two buffers
  static constexpr int oGlo = oGhi + 2 * kGBytes;               // two buffers
  static constexpr int oKz = oGlo + 2 * kGBytes;
  static constexpr int oBar = oKz + kKzSlots * kKzSlotBytes;    // mbarrier, tmem pointer
  static constexpr int oDq = oBar + 16;                         // row-sum terms of two warps
  static constexpr int oS = oDq + 2 * kS2Rows * 16 * 4;         // [16][128] float2 evidence
  static constexpr int oHam = oS + kS2Rows * kS2Threads * 8;    // [4][128] uint2 packed counts
  static constexpr int oK = oHam + 4 * kS2Threads * 8;          // int tables from here
  static constexpr int oKold = oK + kS2Win * 4;
  static constexpr int oVb0 = oKold + kS2Win * 4;
  static constexpr int oVb1 = oVb0 + kS2Win * 4;
  static constexpr int oQ = oVb1 + kS2Win * 4;
  static constexpr int oQold = oQ + kS2Rows * 4;
  static constexpr int oKeep = oQold + kS2Rows * 4;             // [16][8] keep ballots
  static constexpr int oRstat = oKeep + kS2Rows * kVjpWarps * 4;  // [16] float4
  static constexpr int oGlut = oRstat + kS2Rows * 16;           // [64] float
  static constexpr int oUlut = oGlut + 64 * 4;                  // [16][NG][16] float
  static constexpr int kBytes = oUlut + kS2Rows * NG * 16 * 4;
  static_assert(oQz % 16 == 0 && oS % 16 == 0 && oK % 16 == 0 && oRstat % 16 == 0, "alignment");
};


// ---- forward phase: four rows x two diagonals from the running state.  kw / kow hold the key
// symbols (and the symbols leaving the horizon) of window columns cb .. cb + 5, cb the column of
// (row r0, diagonal 1); cell (rr, e) reads entry rr + 1 - e.  Stores S per row and the eight
// mismatch counts (times four: byte offsets into the gate table) as one 64-bit word.  Returns
// whether any window product of the thread may be non-zero.
template <bool kEdge>
__device__ __forceinline__ bool s2_forward_group(const int* s_q, const int* s_qold,
                                                 const float* glut, const int (&kw)[6],
                                                 const int (&kow)[6], bool windowed, int r0, int i0,
                                                 int j1, int W, int len, int hs_cut, float neg_md,
                                                 float (&S)[2], int (&hs)[2], float2* s_row,
                                                 uint2* ham_out) {
  const int4 q4 = *reinterpret_cast<const int4*>(s_q + r0);
  const int q[4] = {q4.x, q4.y, q4.z, q4.w};
  int qo[4] = {0, 0, 0, 0};
  if (windowed) {
    const int4 o4 = *reinterpret_cast<const int4*>(s_qold + r0);
    qo[0] = o4.x; qo[1] = o4.y; qo[2] = o4.z; qo[3] = o4.w;
  }
  int ham[4][2], hsv[4][2];
  bool alive = false;
#pragma unroll
  for (int rr = 0; rr < 4; ++rr)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int x = rr + 1 - e;
      ham[rr][e] = __popc(q[rr] ^ kw[x]);
      hsv[rr][e] = 0;
      if (windowed) {
        const int old = __popc(qo[rr] ^ kow[x]);
        if (kEdge) {
          const int j = j1 + x;
          const bool act = j >= 0 && i0 + r0 + rr <= len - 1;
          hs[e] += act ? ham[rr][e] - (j > W ? old : 0) : 0;
          alive |= j >= W && hs[e] <= hs_cut;
        } else {
          hs[e] += ham[rr][e] - old;
          alive |= hs[e] <= hs_cut;
        }
        hsv[rr][e] = hs[e];
      }
    }
  float P[4][2];
#pragma unroll
  for (int rr = 0; rr < 4; ++rr) P[rr][0] = P[rr][1] = 0.0f;
  const bool any_alive = windowed && __any_sync(0xffffffffu, alive);
  if (any_alive) {
#pragma unroll
    for (int rr = 0; rr < 4; ++rr)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        bool on = hsv[rr][e] <= hs_cut;
        if (kEdge) on = on && (j1 + rr + 1 - e) >= W;
        P[rr][e] = on ? __expf(neg_md * (float)hsv[rr][e]) : 0.0f;
      }
  }
  uint32_t hw[2] = {0u, 0u};
#pragma unroll
  for (int rr = 0; rr < 4; ++rr) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const float x = glut[ham[rr][e]];
      const float Sn = x * (1.0f + S[e]) - P[rr][e];
      bool act = true;
      if (kEdge) act = (j1 + rr + 1 - e) >= 0 && i0 + r0 + rr <= len - 1;
      S[e] = act ? Sn : 0.0f;
      hw[rr >> 1] |= (uint32_t)(ham[rr][e] * 4) << (8 * ((rr & 1) * 2 + e));
    }
    s_row[rr * kS2Threads] = make_float2(S[0], S[1]);
  }
  *ham_out = make_uint2(hw[0], hw[1]);
  return any_alive;
}

// ---- adjoint phase, no window product alive: four rows (descending) x two diagonals.
// sb is the running adjoint of S in float32 (a contraction here), xnext the gate one row
// further down the diagonal.  Writes C and p*d into the operand area.
template <int NG, int NC, int NP, bool kRound, bool kDropout, bool kEdge>
__device__ __forceinline__ void s2_adjoint_group(
    unsigned char* tC, unsigned char* tP, int cg, const float4* s_rstat, uint2 keepw,
    const float* glut, const float* ulut, const uint32_t (&v0)[6], const uint32_t (&v1)[6],
    const float2* s_row, uint2 hamw, int r0, int i0, int j1, int len, int skew, int cb, float mul2,
    int keep_shift, float (&sb)[2], float (&xnext)[2]) {
  // keep flags of the group's four rows, this thread's two diagonals at bits 4 rr, 4 rr + 1
  const uint32_t kgroup = (r0 < 8 ? keepw.x : keepw.y) >> (4 * (r0 & 7) + keep_shift);
  // operand byte offsets of window columns cb .. cb + 4 (cb is even: cb + 1 and cb + 3 never
  // start a new group of eight columns)
  int o[5];
  o[0] = col_off(cb, cg) + row_off(r0);
  o[2] = col_off(cb + 2, cg) + row_off(r0);
  o[4] = col_off(cb + 4, cg) + row_off(r0);
  o[1] = o[0] + 2;
  o[3] = o[2] + 2;
#pragma unroll
  for (int rr = 3; rr >= 0; --rr) {
    const int r = r0 + rr;
    const float4 st = s_rstat[r];          // (exponent bias, 1/Z, E * ds, 1/Z / keep probability)
    const float2 Sv = s_row[rr * kS2Threads];
    const uint32_t hb = rr < 2 ? hamw.x : hamw.y;
    uint32_t kbits = 3u;
    if (kDropout) kbits = kgroup >> (4 * rr);
    float Cv[2], pd[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int x = rr + 1 - e;
      const float Se = e == 0 ? Sv.x : Sv.y;
      const uint32_t hoff = (hb >> (8 * ((rr & 1) * 2 + e))) & 0xffu;
      const float gate = *reinterpret_cast<const float*>(reinterpret_cast<const char*>(glut) + hoff);
      const float t = 1.0f + Se;
      const float rs = rsqrtf(t);
      float ex = exp2f(fmaf(t * rs, mul2, st.x));
      bool act = true;
      if (kEdge) {
        act = (j1 + x) >= 0 && i0 + r <= len - 1;
        ex = act ? ex : 0.0f;
      }
      const float pr = ex * st.y;
      pd[e] = ex * st.w;
      if (kDropout) pd[e] = (kbits >> e & 1u) ? pd[e] : 0.0f;
      else pd[e] = pr;
      const float u = tiled_utility<NG>(ulut + r * NG * 16, v0[x], NG > 4 ? v1[x] : 0u);
      const float dS = (pd[e] * u - pr * st.z) * rs;
      sb[e] = fmaf(xnext[e], sb[e], dS);
      Cv[e] = act ? Se * sb[e] : 0.0f;
      xnext[e] = gate;
    }
    // diagonal 1 sits on the lower column (cb + rr), diagonal 0 on the next one
    const bool aligned = (rr & 1) == 0;
    store_pair<NC, kRound>(tC + rr * 16, o[rr], o[rr + 1], aligned, Cv[1], Cv[0]);
    store_pair<NP, kRound>(tP + rr * 16, o[rr], o[rr + 1], aligned, pd[1], pd[0]);
  }
}

struct S2Geom {
  int w, rb, dmin, dmax, rb_lo, i0, first_row, skew, jwin;
  int64_t ck_idx;
};

// the two variants of the kernel (see the header of the included file)
#include "vjp_tiled_sweep2_kernel.inl"
#define ROSA_S2_PAIR
#include "vjp_tiled_sweep2_kernel.inl"
#undef ROSA_S2_PAIR

template <int NV, int NG, bool kDropout, int kPrec>
int launch_s2_tiled_t(const VjpArgs& a, unsigned grid, cudaStream_t stream) {
  constexpr int bytes = S2Smem<NV, NG, kPrec>::kBytes;
  if constexpr (pairs_blocks(NV)) {
    auto kernel = vjp_sweep2_tiled_pair_kernel<NV, NG, kDropout, kPrec>;
    ROSA_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    kernel<<<grid, kS2Threads, bytes, stream>>>(a);
  } else {
    auto kernel = vjp_sweep2_tiled_kernel<NV, NG, kDropout, kPrec>;
    ROSA_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    kernel<<<grid, kS2Threads, bytes, stream>>>(a);
  }
  ROSA_CUDA_OK(cudaGetLastError());
  return 0;
}

template <int NV, int NG>
int launch_s2_tiled_n(const VjpArgs& a, unsigned grid, cudaStream_t stream) {
  const bool dropout = a.dropout_p > 0.0f;
  const int prec = a.dtype == ROSA_B200_F32 ? 0 : a.dtype == ROSA_B200_F16 ? 1 : 2;
#define ROSA_S2(DO, PR) launch_s2_tiled_t<NV, NG, DO, PR>(a, grid, stream)
  if (dropout) return prec == 0 ? ROSA_S2(true, 0) : prec == 1 ? ROSA_S2(true, 1) : ROSA_S2(true, 2);
  return prec == 0 ? ROSA_S2(false, 0) : prec == 1 ? ROSA_S2(false, 1) : ROSA_S2(false, 2);
#undef ROSA_S2
}

}  // namespace

int launch_vjp_sweep2_tiled(const VjpArgs& a, int items_upper, cudaStream_t stream) {
  const unsigned grid = (unsigned)((int64_t)items_upper * a.H);
  if (a.Dv <= 8) return launch_s2_tiled_n<16, 2>(a, grid, stream);
  if (a.Dv <= 16) return launch_s2_tiled_n<16, 4>(a, grid, stream);
  return launch_s2_tiled_n<32, 8>(a, grid, stream);
}

}  // namespace rosa
