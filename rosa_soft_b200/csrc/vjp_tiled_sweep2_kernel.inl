// Body of the tiled second sweep, included twice by vjp_tiled_sweep2.cu: once as it is
// (vjp_sweep2_tiled_kernel: one block per flush of the column sums, value rows of up to 16
// components) and once with ROSA_S2_PAIR defined (vjp_sweep2_tiled_pair_kernel: two blocks per
// flush, wider value rows).  The two variants are separate expansions of one text rather than
// one template with a constant switch because the unpaired kernel's generated code proved
// sensitive to the mere presence of the pairing logic (62.8 -> 69.3 ms on the long-match
// workload with the switch compiled to "off").
#ifdef ROSA_S2_PAIR
#define S2_TILE_C tCb            /* the cells of the current block inside the 288-column area */
#define S2_TILE_P tPb
#define S2_CHUNK(ch) ((ch) == 2 ? kS2Band - 32 : chunk_start(ch, L::kTileCols))
#define S2_KV_FIRST kv_accumulate /* the second block of a pair adds to the first one's sums */
#else
#define S2_TILE_C tC
#define S2_TILE_P tP
#define S2_CHUNK(ch) ((ch) == 2 ? kS2Band - 32 : chunk_start(ch))
#define S2_KV_FIRST false
#endif

template <int NV, int NG, bool kDropout, int kPrec>
#ifndef ROSA_S2_PAIR
__global__ void __launch_bounds__(kS2Threads, 3) vjp_sweep2_tiled_kernel(VjpArgs a) {
#else /* ROSA_S2_PAIR */
__global__ void __launch_bounds__(kS2Threads) vjp_sweep2_tiled_pair_kernel(VjpArgs a) {
#endif /* ROSA_S2_PAIR */
  using L = S2Smem<NV, NG, kPrec>;
  using TM = Terms<kPrec>;
  constexpr int NC = TM::C, NP = TM::P, CG = L::kCg, NK = kS2NK;
  extern __shared__ float4 smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(smem_raw);
  unsigned char* tC = smem + L::oTile;                    // C terms, kTermBytes apart
  unsigned char* tP = tC + NC * kTermBytes;             // p*d terms
  unsigned char* bKz = smem + L::oKz;
  uint64_t* mbar = reinterpret_cast<uint64_t*>(smem + L::oBar);
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(mbar + 1);
  float* s_dq = reinterpret_cast<float*>(smem + L::oDq);
  float2* Sbuf = reinterpret_cast<float2*>(smem + L::oS);
  uint2* Hbuf = reinterpret_cast<uint2*>(smem + L::oHam);
  int* s_k = reinterpret_cast<int*>(smem + L::oK);
  int* s_kold = reinterpret_cast<int*>(smem + L::oKold);
  uint32_t* s_vb0 = reinterpret_cast<uint32_t*>(smem + L::oVb0);
  uint32_t* s_vb1 = reinterpret_cast<uint32_t*>(smem + L::oVb1);
  int* s_q = reinterpret_cast<int*>(smem + L::oQ);
  int* s_qold = reinterpret_cast<int*>(smem + L::oQold);
  float4* s_rstat = reinterpret_cast<float4*>(smem + L::oRstat);
  float* glut = reinterpret_cast<float*>(smem + L::oGlut);
  float* ulut = reinterpret_cast<float*>(smem + L::oUlut);

  Item it;
  if (!load_item_1d(a, &it)) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool dense = a.plan.cu_seqlens == nullptr;
  const int64_t sym_base = (int64_t)it.seq * a.sym_seq_stride + (int64_t)it.h * a.sym_head_stride +
                           (dense ? 0 : it.start);
  const int32_t* __restrict__ q = a.qsym + sym_base;
  const int32_t* __restrict__ k = a.ksym + sym_base;
  const int vh = it.h / a.group;
  const uint32_t* __restrict__ vb = a.vbits + ((int64_t)vh * a.N + it.start) * a.vwords;
  const int W = a.W, D = a.D, Dv = a.Dv, mask = a.mask, ring_slots = a.ring_slots;
  const bool windowed = ring_slots > 0;
  const float neg_md = -a.mismatch_scale / (float)a.D;
  const int hs_cut = window_sum_cutoff(neg_md);
  const float4* __restrict__ rowstat = a.rowstat + (int64_t)it.h * a.N + it.start;
  float* ring = ring_slots ? a.ring + it.item_linear * (int64_t)ring_slots * kS2Band + kS2R * tid
                           : nullptr;
  constexpr float kLog2e = 1.4426950408889634f;
  const float mul2 = kSqrtScale * a.scale * kLog2e;
  const float ds_mul = a.scale * (0.5f * kSqrtScale);   // folded into the utility tables and E
  constexpr int NQ = 2;                                  // issuers of the row-sum k-loop
  constexpr uint32_t kTmemCols = ((3 + NQ) * NK + 3 * NV) <= 128 ? 128 : 256;
  constexpr uint32_t kColK = 0, kColV = 3 * NK, kColQ = 3 * NK + 3 * NV;
#ifdef ROSA_S2_PAIR
  constexpr bool kPair = pairs_blocks(NV);
#endif /* ROSA_S2_PAIR */

  // ---- one-time set-up
#ifndef ROSA_S2_PAIR
  for (int e = tid; e < operand_bytes(L::kTerms) / 16; e += kS2Threads)
#else /* ROSA_S2_PAIR */
  for (int e = tid; e < operand_bytes(L::kTerms, L::kTileCols) / 16; e += kS2Threads)
#endif /* ROSA_S2_PAIR */
    reinterpret_cast<uint4*>(tC)[e] = make_uint4(0, 0, 0, 0);
  if (tid <= D) glut[tid] = expf(neg_md * (float)tid);
  if (warp == 0) tc::tmem_alloc(tmem_ptr, kTmemCols);
  if (tid == 0) tc::mbar_init(mbar, 4);
  tc::fence_before_thread_sync();
  __syncthreads();
  tc::fence_after_thread_sync();
  const uint32_t tmem = *tmem_ptr;
  uint32_t mma_phase = 0;
  bool mma_timed_out = false;
  int buf = 0;

  auto geom_of = [&](int w, int rb) {
    S2Geom g;
    g.w = w;
    g.rb = rb;
    g.dmin = 1 + w * kS2Band;
    g.dmax = g.dmin + kS2Band - 1;
    g.rb_lo = g.dmin / kS2Rows;
    g.i0 = rb * kS2Rows;
    g.first_row = max(g.i0, g.dmin);
    g.skew = g.first_row - g.i0;
    g.jwin = g.i0 - g.dmax;
    g.ck_idx = it.ck_base + vjp_ck_before(it.len, w) + (rb - g.rb_lo);
    return g;
  };

  // Adds the accumulators of a finished block to the per-item partial gradient rows.  Warp q
  // owns tensor-memory lanes 32 q .. 32 q + 31, i.e. window columns chunk + 32 q + lane of the
  // column sums and one 16-row term slice of the row sums.
#ifdef ROSA_S2_PAIR
  // state of the block whose MMAs are in flight, and of block pairing
  int prev_shift = 0;
  bool prev_flush = true;
  bool pair_first = true;                            // the current block opens a pair of blocks
  // `shift` is 16 for the first block of a pair (its cells sit 16 tile columns up), 0 for the
  // second; `flush`: the pair is complete (or the band ends), the column sums leave tensor memory.
#endif /* ROSA_S2_PAIR */
  auto epilogue = [&](int block_w, int block_rb) {
#ifdef ROSA_S2_PAIR
    // compile-time constants where blocks are not paired
    const int shift = kPair ? prev_shift : 0;
    const bool flush = !kPair || prev_flush;
#endif /* ROSA_S2_PAIR */
    const S2Geom b = geom_of(block_w, block_rb);
#ifdef ROSA_S2_PAIR
    const int jbase = b.jwin - shift;                   // key position of tile column 0
    // blocks whose sums the accumulators hold: this one, and the one above it when it closed a pair
    const int rb_pair_top = block_rb + (kPair && shift == 0 ? 1 : 0);
#endif /* ROSA_S2_PAIR */
    const uint32_t lane_base = (uint32_t)(32 * warp) << 16;
    // where the accumulators of this thread's columns go: worked out before the wait for the
    // tensor core
    float* dst_k[3];
    float* dst_v[3];
    bool use3[3], first3[3];
#pragma unroll
    for (int ch = 0; ch < 3; ++ch) {
#ifndef ROSA_S2_PAIR
      const int c = S2_CHUNK(ch) + 32 * warp + lane;
      const int j = b.jwin + c;
      // the last chunk starts at column 224, past-the-window columns included (its MMA reads
      // on into the B operand buffers; those lanes are never used): its new columns 256..271
      // fall into the second lane quarter, whose warp has the shortest MMA issue list
      use3[ch] = (ch < 2 || (warp == 1 && c >= 256 && c < kS2Win)) && j >= 0 && j <= it.len - 1 - b.dmin;
      const int i_top = min(j + b.dmax, it.len - 1);
      const bool first = (b.w == it.w_begin) && (b.rb == i_top / kS2Rows);
#else /* ROSA_S2_PAIR */
      const int c = S2_CHUNK(ch) + 32 * warp + lane;
      const int j = jbase + c;
      // only tile columns >= 256 of the last chunk (which starts at column 224) are new: they sit
      // in the second lane quarter
      use3[ch] = flush && (ch < 2 || (warp == 1 && c >= 256 && c < L::kTileCols)) && j >= 0 &&
                 j <= it.len - 1 - b.dmin;
      // the first block of the item that holds column j: the flush of its pair stores, later
      // ones add
      const int rb_first = min(j + b.dmax, it.len - 1) / kS2Rows;
      const bool first = (b.w == it.w_begin) &&
                         (kPair ? rb_first <= rb_pair_top && rb_first >= b.rb : rb_first == b.rb);
#endif /* ROSA_S2_PAIR */
      first3[ch] = first;
      dst_k[ch] = a.dk_part + (it.rowslot + j) * D;
      dst_v[ch] = a.dv_part + (it.rowslot + j + 1) * Dv;
    }
    if (!mma_timed_out && !__all_sync(0xffffffffu, tc::mbar_wait(mbar, mma_phase, 1u << 24)))
      mma_timed_out = true;
    if (mma_timed_out) {   // nothing accumulated may be trusted; keep the named barrier whole
      if ((mask & 1) && warp < NC) asm volatile("bar.sync 1, %0;" ::"n"(32 * NC) : "memory");
      return;
    }
    mma_phase ^= 1u;
    tc::fence_after_thread_sync();
#ifdef ROSA_S2_PAIR
    if (flush)       // the first block of a pair leaves its column sums in tensor memory
#endif
#pragma unroll
    for (int ch = 0; ch < 3; ++ch) {
      if (ch == 2 && warp != 1) continue;
      const bool use = use3[ch], first = first3[ch];
      if (mask & 2) {
        float v[16];
        tc::tmem_ld16(tmem + lane_base + kColK + ch * NK, v);
        if (use) {
          float* dst = dst_k[ch];
          if ((D & 3) == 0) {
#pragma unroll
            for (int d4 = 0; d4 < 4; ++d4)
              if (4 * d4 < D) {
                float4* p4 = reinterpret_cast<float4*>(dst) + d4;
                accumulate_row4(p4, first, v[4 * d4], v[4 * d4 + 1], v[4 * d4 + 2], v[4 * d4 + 3]);
              }
          } else {
#pragma unroll
            for (int d = 0; d < 16; ++d)
              if (d < D) accumulate_row1(dst + d, first, v[d]);
          }
        }
      }
      if (mask & 4) {
#pragma unroll
        for (int n0 = 0; n0 < NV; n0 += 16) {
          float v[16];
          tc::tmem_ld16(tmem + lane_base + kColV + ch * NV + n0, v);
          if (use && n0 < Dv) {
            float* dst = dst_v[ch] + n0;
            if ((Dv & 3) == 0) {
#pragma unroll
              for (int d4 = 0; d4 < 4; ++d4)
                if (n0 + 4 * d4 < Dv) {
                  float4* p4 = reinterpret_cast<float4*>(dst) + d4;
                  accumulate_row4(p4, first, v[4 * d4], v[4 * d4 + 1], v[4 * d4 + 2], v[4 * d4 + 3]);
                }
            } else {
#pragma unroll
              for (int d = 0; d < 16; ++d)
                if (n0 + d < Dv) accumulate_row1(dst + d, first, v[d]);
            }
          }
        }
      }
    }
    if ((mask & 1) && warp < NC) {
      // accumulator rows 16 t .. 16 t + 15 (term t of C) sit in lanes 0-15 of lane quarter t
      float v[16], v2[16];
      tc::tmem_ld16(tmem + lane_base + kColQ, v);
      tc::tmem_ld16(tmem + lane_base + kColQ + NK, v2);
#pragma unroll
      for (int d = 0; d < 16; ++d) v[d] += v2[d];
      if (warp > 0 && lane < kS2Rows) {
        float4* dst4 = reinterpret_cast<float4*>(s_dq + ((warp - 1) * kS2Rows + lane) * 16);
#pragma unroll
        for (int d4 = 0; d4 < 4; ++d4)
          dst4[d4] = make_float4(v[4 * d4], v[4 * d4 + 1], v[4 * d4 + 2], v[4 * d4 + 3]);
      }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * NC) : "memory");
      const int i = b.i0 + lane;
      if (warp == 0 && lane < kS2Rows && i >= b.first_row && i <= it.len - 1) {
        float* dst = a.dq_part + (it.rowslot + i) * D;
#pragma unroll
        for (int d4 = 0; d4 < 4; ++d4) {
          if (4 * d4 >= D) break;
          float sum[4] = {v[4 * d4], v[4 * d4 + 1], v[4 * d4 + 2], v[4 * d4 + 3]};
#pragma unroll
          for (int t = 1; t < NC; ++t) {
            const float4 o =
                *reinterpret_cast<const float4*>(s_dq + ((t - 1) * kS2Rows + lane) * 16 + 4 * d4);
            sum[0] += o.x; sum[1] += o.y; sum[2] += o.z; sum[3] += o.w;
          }
          if ((D & 3) == 0) {
            accumulate_row4(reinterpret_cast<float4*>(dst) + d4, b.w == it.w_begin, sum[0], sum[1],
                            sum[2], sum[3]);
          } else {
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              const int d = 4 * d4 + x;
              if (d < D) accumulate_row1(dst + d, b.w == it.w_begin, sum[x]);
            }
          }
        }
      }
    }
    tc::fence_before_thread_sync();
  };

  const int rb_top = (it.len - 1) / kS2Rows;     // bottom row block of every band
  const float inv_keep = a.inv_keep;
  const int keep_shift = 2 * (tid & 1);

  // Tables of one block: column windows, row symbols and statistics, keep ballots, utility
  // tables (scaled by ds_mul: the adjoint seed then needs no further factor), the grad_output
  // operand of the value sums and the thread's checkpoints.  They are fetched in two steps: the
  // global loads of block b + 1 are issued into registers before the adjoint phase of block b
  // and stored to shared memory after it, so their latency is never waited for.
  constexpr int kColRegs = (kS2Win + kS2Threads - 1) / kS2Threads;        // 3
  constexpr int kGoRegs = (NV * kS2Rows + kS2Threads - 1) / kS2Threads;   // 2 or 4
  struct Prefetch {
    int k[kColRegs], kold[kColRegs];
    uint32_t vb[kColRegs];
    int q, qold;
    float4 st;
    uint2 keep;            // keep flags of the sweep-1 thread that owns these two diagonals
    uint32_t lut[4];       // raw grad_output elements of this thread's (row, value group)
    uint32_t go[kGoRegs];  // raw grad_output elements of the operand tile
    int4 ck;
  };
  auto go_bits = [&](int i, int d) -> uint32_t {
    const int64_t idx = (((int64_t)it.start + i) * a.H + it.h) * Dv + d;
    return a.dtype == ROSA_B200_F32 ? static_cast<const uint32_t*>(a.go)[idx]
                                    : (uint32_t) static_cast<const uint16_t*>(a.go)[idx];
  };
  auto go_float = [&](uint32_t bits) {
    if (a.dtype == ROSA_B200_F32) return __uint_as_float(bits);
    if (a.dtype == ROSA_B200_F16) return __half2float(__ushort_as_half((unsigned short)bits));
    return __uint_as_float(bits << 16);          // bf16 is the upper half of a float
  };
  auto prefetch_load = [&](const S2Geom& g, Prefetch& pf) {
#pragma unroll
    for (int x = 0; x < kColRegs; ++x) {
      const int c = tid + x * kS2Threads;
      const int j = g.jwin + c;
      const bool in = c < kS2Win && j >= 0 && j < it.len - 1;
      pf.k[x] = in ? __ldg(k + j) : 0;
      const int jo = j - W - 1;
      pf.kold[x] = (windowed && c < kS2Win && jo >= 0 && jo < it.len) ? __ldg(k + jo) : 0;
      pf.vb[x] = in ? __ldg(vb + j + 1) : 0u;
    }
    pf.q = pf.qold = 0;
    pf.st = make_float4(0.f, 0.f, 0.f, 0.f);
    if (tid < kS2Rows) {
      const int i = g.i0 + tid;
      if (i >= g.first_row && i <= it.len - 1) {
        pf.q = __ldg(q + i);
        if (windowed && i - W - 1 >= 0) pf.qold = __ldg(q + i - W - 1);
        pf.st = rowstat[i];                          // (max, 1/Z, E, log i)
      }
    }
    pf.keep = make_uint2(0u, 0u);
    if (kDropout)   // word of sweep-1 thread tid / 2: row r, diagonal e of that thread at bit 4 r + e
      pf.keep = reinterpret_cast<const uint2*>(a.keepbits)[g.ck_idx * (kS2Band / 4) + (tid >> 1)];
#pragma unroll
    for (int b = 0; b < 4; ++b) pf.lut[b] = 0u;
    if (tid < kS2Rows * NG) {
      const int r = tid / NG, gq = tid - r * NG;
      const int i = g.i0 + r;
      if (i >= g.first_row && i <= it.len - 1) {
#pragma unroll
        for (int b = 0; b < 4; ++b)
          if (4 * gq + b < Dv) pf.lut[b] = go_bits(i, 4 * gq + b);
      }
    }
#pragma unroll
    for (int x = 0; x < kGoRegs; ++x) {
      const int e = tid + x * kS2Threads;
      const int d = e / kS2Rows, r = e - d * kS2Rows;
      const int i = g.i0 + r;
      pf.go[x] = 0u;
      if ((mask & 4) && e < NV * kS2Rows && d < Dv && i >= g.first_row && i <= it.len - 1)
        pf.go[x] = go_bits(i, d);
    }
    pf.ck = *reinterpret_cast<const int4*>(a.ckpt + g.ck_idx * kS2Band + kS2R * tid);
  };
  auto prefetch_store = [&](const Prefetch& pf, unsigned char* bGhi, unsigned char* bGlo) {
#pragma unroll
    for (int x = 0; x < kColRegs; ++x) {
      const int c = tid + x * kS2Threads;
      if (c < kS2Win) {
        s_k[c] = pf.k[x];
        s_kold[c] = pf.kold[x];
        s_vb0[c] = spread_nibbles(pf.vb[x] & 0xffffu);
        if (NG > 4) s_vb1[c] = spread_nibbles(pf.vb[x] >> 16);
      }
    }
    if (tid < kS2Rows) {
      s_q[tid] = pf.q;
      s_qold[tid] = pf.qold;
      s_rstat[tid] = make_float4(-(pf.st.w + pf.st.x) * kLog2e - mul2, pf.st.y, pf.st.z * ds_mul,
                                 pf.st.y * inv_keep);
    }
    if (tid < kS2Rows * NG) {
      float gv[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) gv[b] = ds_mul * go_float(pf.lut[b]);
      float4* dst = reinterpret_cast<float4*>(ulut + tid * 16);
#pragma unroll
      for (int n4 = 0; n4 < 4; ++n4) {
        const float hi = ((n4 & 1) ? gv[2] : -gv[2]) + ((n4 & 2) ? gv[3] : -gv[3]);
        dst[n4] = make_float4(hi - gv[0] - gv[1], hi + gv[0] - gv[1], hi - gv[0] + gv[1],
                              hi + gv[0] + gv[1]);
      }
    }
    if (mask & 4) {
#pragma unroll
      for (int x = 0; x < kGoRegs; ++x) {
        const int e = tid + x * kS2Threads;
        if (e < NV * kS2Rows) {
          const int d = e / kS2Rows, r = e - d * kS2Rows;
          const float v = go_float(pf.go[x]);
          const __nv_bfloat16 h = __float2bfloat16_rn(v);
          *reinterpret_cast<__nv_bfloat16*>(bGhi + b_off(d, r, NV)) = h;
          if (TM::glo)
            *reinterpret_cast<__nv_bfloat16*>(bGlo + b_off(d, r, NV)) =
                __float2bfloat16_rn(v - __bfloat162float(h));
        }
      }
    }
  };

  int w = it.w_begin, rb = rb_top;
  int prev_w = 0, prev_rb = 0;
  bool prev_pending = false, band_start = true;
  // per-band state of the thread's two diagonals
  float sb[2] = {0.f, 0.f}, xnext[2] = {0.f, 0.f};
  double Sbar[2] = {0.0, 0.0}, Y[2] = {0.0, 0.0};
  int live = 0;
  bool ring_dirty = false;
  Prefetch pf;
  {
    prefetch_load(geom_of(w, rb), pf);
    prefetch_store(pf, smem + L::oGhi, smem + L::oGlo);
    __syncthreads();
  }
  int4 ck = pf.ck;
  uint2 keepw = pf.keep;

  while (true) {
    const S2Geom g = geom_of(w, rb);
    const int delta0 = g.dmin + kS2R * tid;            // diagonal of e = 0
    if (band_start) {
      sb[0] = sb[1] = xnext[0] = xnext[1] = 0.0f;
      Sbar[0] = Sbar[1] = Y[0] = Y[1] = 0.0;
      live = 0;
      ring_dirty = false;
      // the bottom block of a band refills the whole kz^T ring: the last block of the previous
      // band must have released it
      if (prev_pending) {
        epilogue(prev_w, prev_rb);
        prev_pending = false;
      }
    }
    const bool next_same = rb > g.rb_lo;
    const bool has_next = next_same || w + 1 < it.w_end;
#ifdef ROSA_S2_PAIR
    if (kPair && band_start) pair_first = true;
    const int tile_shift = kPair && pair_first ? kS2Rows : 0;      // tile column of window column 0
    const bool flush = !kPair || !pair_first || !next_same;      // the pair (or the band) ends here
    const bool kv_accumulate = kPair && !pair_first;   // second block of a pair
    unsigned char* tCb = tC + (tile_shift >> 3) * CG;  // this block's cells
    unsigned char* tPb = tP + (tile_shift >> 3) * CG;
#endif /* ROSA_S2_PAIR */
    unsigned char* bQz = smem + L::oQz + buf * L::kQzBytes;
    unsigned char* bGhi = smem + L::oGhi + buf * L::kGBytes;
    unsigned char* bGlo = smem + L::oGlo + buf * L::kGBytes;

    (void)bGhi;
    (void)bGlo;
    // ---- B operands that come from the tables
    if (mask & 2)
      for (int e = tid; e < NK * kS2Rows; e += kS2Threads) {
        const int d = e / kS2Rows, r = e - d * kS2Rows;
        const int i = g.i0 + r;
        const float v = (d < D && i >= g.first_row && i <= it.len - 1)
                            ? ((s_q[r] >> d & 1) ? 1.0f : -1.0f) : 0.0f;
        *reinterpret_cast<__nv_bfloat16*>(bQz + b_off(d, r, NK)) = __float2bfloat16_rn(v);
      }
    if (mask & 1) {
      const int g0 = (g.jwin + (1 << 20)) >> 4;        // absolute group of window column 0
      const int nfill = band_start ? kS2Win / 16 : 1;
      for (int e = tid; e < nfill * NK * 16; e += kS2Threads) {
        const int ks = e / (NK * 16), rem = e - ks * (NK * 16);
        const int d = rem >> 4, cc = rem & 15;
        const int c = ks * 16 + cc;
        const int j = g.jwin + c;
        const float v = (d < D && j >= 0 && j < it.len - 1)
                            ? ((s_k[c] >> d & 1) ? 1.0f : -1.0f) : 0.0f;
        const int sl = (g0 + ks) % L::kKzSlots;
        *reinterpret_cast<__nv_bfloat16*>(bKz + sl * L::kKzSlotBytes + b_off(d, cc, NK)) =
            __float2bfloat16_rn(v);
      }
    }

    // ---- phase A: forward recurrence of the block from its checkpoint
    float S[2] = {__int_as_float(ck.x), __int_as_float(ck.z)};
    int hs[2] = {ck.y, ck.w};
    const bool interior = g.jwin >= (windowed ? W + 1 : 0) && g.i0 + kS2Rows - 1 <= it.len - 1;
    const int cb0 = kS2Band - 2 - kS2R * tid;          // window column of (row 0, diagonal 1)
    bool has_p = false;
    {
      int kw[6], kow[6] = {0, 0, 0, 0, 0, 0};
      const int2 a0 = *reinterpret_cast<const int2*>(s_k + cb0);
      kw[0] = a0.x; kw[1] = a0.y;
      if (windowed) {
        const int2 b0 = *reinterpret_cast<const int2*>(s_kold + cb0);
        kow[0] = b0.x; kow[1] = b0.y;
      }
#pragma unroll 1
      for (int r0 = 0; r0 < kS2Rows; r0 += 4) {
        const int cb = cb0 + r0;
        const int2 a1 = *reinterpret_cast<const int2*>(s_k + cb + 2);
        const int2 a2 = *reinterpret_cast<const int2*>(s_k + cb + 4);
        kw[2] = a1.x; kw[3] = a1.y; kw[4] = a2.x; kw[5] = a2.y;
        if (windowed) {
          const int2 b1 = *reinterpret_cast<const int2*>(s_kold + cb + 2);
          const int2 b2 = *reinterpret_cast<const int2*>(s_kold + cb + 4);
          kow[2] = b1.x; kow[3] = b1.y; kow[4] = b2.x; kow[5] = b2.y;
        }
        const int j1 = g.jwin + cb;                    // key column of (row r0, diagonal 1)
        float2* s_row = Sbuf + r0 * kS2Threads + tid;
        uint2* ham_out = Hbuf + (r0 >> 2) * kS2Threads + tid;
        if (interior)
          has_p |= s2_forward_group<false>(s_q, s_qold, glut, kw, kow, windowed, r0, g.i0, j1, W,
                                           it.len, hs_cut, neg_md, S, hs, s_row, ham_out);
        else
          has_p |= s2_forward_group<true>(s_q, s_qold, glut, kw, kow, windowed, r0, g.i0, j1, W,
                                          it.len, hs_cut, neg_md, S, hs, s_row, ham_out);
        kw[0] = kw[4]; kw[1] = kw[5];
        kow[0] = kow[4]; kow[1] = kow[5];
      }
    }

    // ---- the next block's tables start their way from global memory now
    if (has_next) prefetch_load(next_same ? geom_of(w, rb - 1) : geom_of(w + 1, rb_top), pf);

    // ---- the previous block's MMAs have had the whole table / forward phase to finish
    if (prev_pending) epilogue(prev_w, prev_rb);

#ifdef ROSA_S2_PAIR
    // ---- the 16 x 16 strip that the other block of the pair filled and this one leaves alone
    // (row r: tile columns r .. r + 15 for the first block of a pair, r + 256 .. r + 271 for the
    // second) is cleared, two cells per thread and term
    if (kPair) {
      const int r = tid >> 3;
      const int c = (pair_first ? 0 : kS2Band) + r + 2 * (tid & 7);
      const int off_lo = col_off(c, CG) + row_off(r), off_hi = col_off(c + 1, CG) + row_off(r);
#pragma unroll
      for (int t = 0; t < NC + NP; ++t) {
        unsigned char* base = tC + t * kTermBytes;
        if ((r & 1) == 0) {
          *reinterpret_cast<uint32_t*>(base + off_lo) = 0u;
        } else {
          *reinterpret_cast<uint16_t*>(base + off_lo) = 0;
          *reinterpret_cast<uint16_t*>(base + off_hi) = 0;
        }
      }
    }

#endif /* ROSA_S2_PAIR */
    // ---- phase B: adjoint recurrence, rows descending; C and p*d go to the operand area
    const bool warp_p = windowed && ring != nullptr && has_p;
    if (!warp_p && live == 0) {
      sb[0] = (float)Sbar[0];
      sb[1] = (float)Sbar[1];
      uint32_t v0[6], v1[6] = {0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll 1
      for (int r0 = kS2Rows - 4; r0 >= 0; r0 -= 4) {
        const int cb = cb0 + r0;
#pragma unroll
        for (int x2 = 0; x2 < 3; ++x2) {
          const uint2 t0 = *reinterpret_cast<const uint2*>(s_vb0 + cb + 2 * x2);
          v0[2 * x2] = t0.x; v0[2 * x2 + 1] = t0.y;
          if (NG > 4) {
            const uint2 t1 = *reinterpret_cast<const uint2*>(s_vb1 + cb + 2 * x2);
            v1[2 * x2] = t1.x; v1[2 * x2 + 1] = t1.y;
          }
        }
        const float2* s_row = Sbuf + r0 * kS2Threads + tid;
        const uint2 hamw = Hbuf[(r0 >> 2) * kS2Threads + tid];
        const int j1 = g.jwin + cb;
        if (interior)
          s2_adjoint_group<NG, NC, NP, kPrec == 0, kDropout, false>(S2_TILE_C, S2_TILE_P, CG, s_rstat, keepw, glut, ulut, v0,
                                                        v1, s_row, hamw, r0, g.i0, j1, it.len,
                                                        g.skew, cb, mul2, keep_shift, sb, xnext);
        else
          s2_adjoint_group<NG, NC, NP, kPrec == 0, kDropout, true>(S2_TILE_C, S2_TILE_P, CG, s_rstat, keepw, glut, ulut, v0,
                                                       v1, s_row, hamw, r0, g.i0, j1, it.len,
                                                       g.skew, cb, mul2, keep_shift, sb, xnext);
      }
      Sbar[0] = (double)sb[0];
      Sbar[1] = (double)sb[1];
    } else {
      // A window product is (or recently was) alive in this warp.  The product is rebuilt from
      // the mismatch-count sum walked backwards (hs ended phase A on the block's last row); the
      // sliding sum Y of Sbar * P over W + 1 rows lives in a ring indexed by the row, so a warp
      // reads and writes one contiguous line per row.
      int slot = (g.i0 + kS2Rows - 1) % ring_slots;    // ring line of the row, walked downwards
#pragma unroll 1
      for (int r = kS2Rows - 1; r >= 0; --r) {
        const int i = g.i0 + r;
        const float4 st = s_rstat[r];
        const float2 Sv2 = Sbuf[r * kS2Threads + tid];
        const uint2 hamw = Hbuf[(r >> 2) * kS2Threads + tid];
        const uint32_t hb = (r & 3) < 2 ? hamw.x : hamw.y;
        uint32_t kbits = 3u;
        if (kDropout) kbits = (r < 8 ? keepw.x : keepw.y) >> (4 * (r & 7) + keep_shift);
        const int qo = s_qold[r];
        float Cv[2], pd[2], Pv[2], gate[2], dS[2];
        bool act[2];
        // the ring line of this row is requested first: while no window product has been alive
        // for W + 2 rows the ring holds zeros and nothing is read
        float* line = ring + (int64_t)slot * kS2Band;
        slot = (slot == 0 ? ring_slots : slot) - 1;
        float2 old_t = make_float2(0.0f, 0.0f);
        if (live > 0) old_t = *reinterpret_cast<const float2*>(line);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int c = r + kS2Band - 1 - kS2R * tid - e;
          const int j = g.jwin + c;
          act[e] = j >= 0 && i <= it.len - 1;
          const uint32_t hoff = (hb >> (8 * ((r & 1) * 2 + e))) & 0xffu;
          const int ham = (int)(hoff >> 2);
          gate[e] = glut[ham];
          Pv[e] = (act[e] && j >= W) ? __expf(neg_md * (float)hs[e]) : 0.0f;
          hs[e] += ((act[e] && j > W) ? __popc(qo ^ s_kold[c]) : 0) - (act[e] ? ham : 0);
          const float Se = e == 0 ? Sv2.x : Sv2.y;
          const float t = 1.0f + Se;
          const float rs = rsqrtf(t);
          const float ex = act[e] ? exp2f(fmaf(t * rs, mul2, st.x)) : 0.0f;
          const float pr = ex * st.y;
          pd[e] = ex * st.w;
          if (kDropout) pd[e] = (kbits >> e & 1u) ? pd[e] : 0.0f;
          const float u = tiled_utility<NG>(ulut + r * NG * 16, s_vb0[c], NG > 4 ? s_vb1[c] : 0u);
          dS[e] = (pd[e] * u - pr * st.z) * rs;
          if (act[e]) Sbar[e] = (double)dS[e] + (double)xnext[e] * Sbar[e];
        }
        const bool any_p = __any_sync(0xffffffffu, Pv[0] != 0.0f || Pv[1] != 0.0f);
        if (any_p) {
          live = W + 2;
          ring_dirty = true;
        }
        if (live > 0) {
#pragma unroll
          for (int e = 0; e < 2; ++e)
            if (act[e]) {
              const float tf = (float)(Sbar[e] * (double)Pv[e]);
              const float old = e == 0 ? old_t.x : old_t.y;
              line[e] = tf;
              Y[e] += (double)tf - (double)old;
            }
          if (--live == 0) Y[0] = Y[1] = 0.0;
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float Se = e == 0 ? Sv2.x : Sv2.y;
          Cv[e] = act[e] ? (float)((double)(Se + Pv[e]) * Sbar[e] - Y[e]) : 0.0f;
          if (act[e]) xnext[e] = gate[e];
        }
        const int c1 = r + kS2Band - 2 - kS2R * tid;           // column of diagonal 1
        const int off_lo = col_off(c1, CG) + row_off(r), off_hi = col_off(c1 + 1, CG) + row_off(r);
        if ((r & 1) == 0) {
          store_pair<NC, kPrec == 0>(S2_TILE_C, off_lo, off_hi, true, Cv[1], Cv[0]);
          store_pair<NP, kPrec == 0>(S2_TILE_P, off_lo, off_hi, true, pd[1], pd[0]);
        } else {
          store_pair<NC, kPrec == 0>(S2_TILE_C, off_lo, off_hi, false, Cv[1], Cv[0]);
          store_pair<NP, kPrec == 0>(S2_TILE_P, off_lo, off_hi, false, pd[1], pd[0]);
        }
      }
    }
    (void)delta0;

    // ---- the tables of the next block replace this block's once every warp is done with them
    __syncthreads();
    if (has_next) {
      prefetch_store(pf, smem + L::oGhi + (buf ^ 1) * L::kGBytes,
                     smem + L::oGlo + (buf ^ 1) * L::kGBytes);
      ck = pf.ck;
    }
    keepw = pf.keep;

    // ---- phase C: hand the operands to the tensor core
    tc::fence_proxy_async_smem();
    tc::fence_before_thread_sync();
    __syncthreads();                               // sync 2: tiles and B operands complete
    if (lane == 0 && !mma_timed_out) {
      tc::fence_after_thread_sync();
      constexpr uint32_t idK = tc::idesc_bf16_f32(128, NK, true, false);
      constexpr uint32_t idV = tc::idesc_bf16_f32(128, NV, true, false);
      constexpr uint32_t idQ = tc::idesc_bf16_f32(64, NK, false, false);
      if (warp == 0 && (mask & 2)) {
        const uint64_t dQz = tc::smem_desc(tc::smem_addr(bQz), NK / 8 * 128, 128);
        const uint64_t c0 = tc::smem_desc(tc::smem_addr(tC), kRowGroupBytes, CG);
        const uint64_t c1 = tc::smem_desc(tc::smem_addr(tC + kTermBytes), kRowGroupBytes, CG);
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) {
          const uint64_t shift = (uint64_t)(((S2_CHUNK(ch) >> 3) * CG) >> 4);
          tc::mma_bf16(tmem + kColK + ch * NK, c0 + shift, dQz, idK, S2_KV_FIRST);
          tc::mma_bf16(tmem + kColK + ch * NK, c1 + shift, dQz, idK, true);
        }
      }
      if (warp == 1 && (mask & 4)) {
        const uint64_t dGhi = tc::smem_desc(tc::smem_addr(bGhi), NV / 8 * 128, 128);
        const uint64_t dGlo = tc::smem_desc(tc::smem_addr(bGlo), NV / 8 * 128, 128);
        const uint64_t p0 = tc::smem_desc(tc::smem_addr(tP), kRowGroupBytes, CG);
        const uint64_t p1 = tc::smem_desc(tc::smem_addr(tP + kTermBytes), kRowGroupBytes, CG);
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) {
          const uint64_t shift = (uint64_t)(((S2_CHUNK(ch) >> 3) * CG) >> 4);
          tc::mma_bf16(tmem + kColV + ch * NV, p0 + shift, dGhi, idV, S2_KV_FIRST);
          if (NP == 2) tc::mma_bf16(tmem + kColV + ch * NV, p1 + shift, dGhi, idV, true);
          if (TM::glo) tc::mma_bf16(tmem + kColV + ch * NV, p0 + shift, dGlo, idV, true);
        }
      }
      if (warp >= 2 && (mask & 1)) {
        // K-major view (row sums): K direction = column groups, M direction = the row groups of
        // the C terms of a column group (M = 64: the rows past the last term alias p*d cores)
        const uint64_t kC = tc::smem_desc(tc::smem_addr(S2_TILE_C), CG, kRowGroupBytes);
        const uint64_t dKz0 = tc::smem_desc(tc::smem_addr(bKz), NK / 8 * 128, 128);
        constexpr int kSteps = kS2Win / 16;
        const int part = warp - 2;
        const int ks0 = part * kSteps / NQ, ks1 = (part + 1) * kSteps / NQ;
        const uint32_t acc = tmem + kColQ + part * NK;
        const int g0 = (g.jwin + (1 << 20)) >> 4;
        int sl = (g0 + ks0) % L::kKzSlots;
#pragma unroll 1
        for (int ks = ks0; ks < ks1; ++ks) {
          const uint64_t dKz = dKz0 + (uint64_t)((sl * L::kKzSlotBytes) >> 4);
          const uint64_t shift = (uint64_t)((ks * 2 * CG) >> 4);
          tc::mma_bf16(acc, kC + shift, dKz, idQ, ks > ks0);
          sl = sl + 1 == L::kKzSlots ? 0 : sl + 1;
        }
      }
      tc::mma_commit(mbar);
    }
    prev_w = w;
    prev_rb = rb;
    prev_pending = true;
#ifdef ROSA_S2_PAIR
    if (kPair) {
      prev_shift = tile_shift;
      prev_flush = flush;
      pair_first = flush;                            // a flushed pair is followed by a new one
    }
#endif /* ROSA_S2_PAIR */
    buf ^= 1;
    // leave the ring zeroed for the next band of this item
    if (!next_same && ring != nullptr && ring_dirty && has_next)
      for (int sl = 0; sl < ring_slots; ++sl) {
        ring[(int64_t)sl * kS2Band] = 0.0f;
        ring[(int64_t)sl * kS2Band + 1] = 0.0f;
      }
    if (!has_next) break;
    band_start = !next_same;
    if (next_same) {
      --rb;
    } else {
      ++w;
      rb = rb_top;
    }
  }
  if (prev_pending) epilogue(prev_w, prev_rb);
  __syncthreads();
  if (mma_timed_out && lane == 0) atomicExch(a.plan.status + 1, 1);
  if (warp == 0) tc::tmem_dealloc(tmem, kTmemCols);
}

#undef S2_TILE_C
#undef S2_TILE_P
#undef S2_CHUNK
#undef S2_KV_FIRST
