// Latent attention in bfloat16 on the tensor cores (mma.sync m16n8k16, float32 accumulation), prompt portions and
// decoded tokens alike.  All heads of a request read the same cache entries [c | kr] (R + P numbers), so the rows
// of a tile are (token, head) pairs: row = token * H + head, 64 rows per CTA, and one pass over the request's
// entries serves every head.  Per tile of 32 entries:
//
//   S = Q K^T over all R + P numbers (the entry is the key), scaled, causal mask, to shared memory in float32;
//   online softmax in float32, four threads per row; the weights are left as TWO bfloat16 numbers, the rounded
//   weight and the rounding's remainder, so that the product with the values carries them to 2^-17;
//   O += P_hi V + P_lo V with V the first R numbers of the same tile, each warp owning 16 rows and half of R.
//
// Entries arrive by cp.async, two tiles in flight.  With n_splits > 1 (decode: few rows, many entries) CTA z takes
// the z-th share of the key tiles and leaves (max, sum, unnormalised output) for the join kernel, which adds the
// shares in their order.  How the tiles are cut into shares follows from the request's length, read on the device.
#include "common.cuh"
#include <math.h>
using namespace bspec;

namespace {

constexpr int BM = 64, BN = 32, THREADS = 256;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__host__ __device__ inline size_t smem_bytes(int D) {
  const int DP = D + 8;
  return (size_t)(BM + 2 * BN) * DP * 2 + (size_t)BM * (BN + 1) * 4 + 2 * (size_t)BM * (BN + 8) * 2 + 3 * BM * 4;
}

// NT: n-tiles (of 8 columns) of the output that one warp may own: R / 16 <= NT.
template <int NT>
__global__ void __launch_bounds__(THREADS)
latent_attn_mma_kernel(const __nv_bfloat16* __restrict__ ql, long long ql_row, long long ql_head,
                       const __nv_bfloat16* __restrict__ qr, long long qr_row, long long qr_head,
                       __nv_bfloat16* __restrict__ out, long long o_row, long long o_head,
                       const __nv_bfloat16* __restrict__ cache, const int* __restrict__ qo_indptr,
                       const int* __restrict__ positions, const int* __restrict__ kv_indptr,
                       const int* __restrict__ kv_indices, int H, int R, int P, int page_size, float scale,
                       int n_splits, float* __restrict__ o_part, float* __restrict__ ml_part, long long n_pages,
                       const float* __restrict__ inv_freq, float magnitude) {
  bspec::pdl_prologue(43);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = R + P, DP = D + 8, PP = BN + 8, SP = BN + 1;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Ks = Qs + (size_t)BM * DP;
  float* Ss = reinterpret_cast<float*>(Ks + (size_t)2 * BN * DP);
  __nv_bfloat16* Ph = reinterpret_cast<__nv_bfloat16*>(Ss + (size_t)BM * SP);
  __nv_bfloat16* Pl = Ph + (size_t)BM * PP;
  float* row_m = reinterpret_cast<float*>(Pl + (size_t)BM * PP);
  float* row_l = row_m + BM;
  float* row_c = row_l + BM;

  const int e = blockIdx.y, split = blockIdx.z;
  const int q_begin = qo_indptr[e], q_len = qo_indptr[e + 1] - q_begin;
  const long long rows_total = (long long)q_len * H;
  const long long row0 = (long long)blockIdx.x * BM;
  if (row0 >= rows_total) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp & 3, ch = warp >> 2;
  const int pos0 = positions[q_begin];
  const int last_tok = (int)min((long long)q_len - 1, (row0 + BM - 1) / H);
  const int max_pos = pos0 + last_tok;
  const int n_tiles = max_pos / BN + 1;
  const int per = (n_tiles + n_splits - 1) / n_splits;
  const int t_begin = split * per, t_end = min(n_tiles, t_begin + per);
  const int* table = kv_indices + kv_indptr[e];

  // ---- queries: row r holds [ql | qr] of (token, head) = divmod(row0 + r, H); rows past the portion are zero.
  // With a frequency table the rotated part arrives unrotated and is rotated here (adjacent pairs, the angle in
  // float64 from the two-float frequencies, cosine and sine times the magnitude), then rounded as a separate
  // rotation kernel would have left it.
  for (int idx = tid; idx < BM * (D / 2); idx += THREADS) {
    const int r = idx / (D / 2), d = 2 * (idx - r * (D / 2));
    const long long row = row0 + r;
    float u = 0.f, v = 0.f;
    if (row < rows_total) {
      const long long t = q_begin + row / H;
      const int h = (int)(row % H);
      if (d < R) {
        const __nv_bfloat16* src = ql + t * ql_row + h * ql_head + d;
        u = __bfloat162float(src[0]);
        v = __bfloat162float(src[1]);
      } else {
        const __nv_bfloat16* src = qr + t * qr_row + h * qr_head + (d - R);
        u = __bfloat162float(src[0]);
        v = __bfloat162float(src[1]);
        if (inv_freq != nullptr) {
          const int j = (d - R) / 2, half = P / 2;
          const double f = (double)inv_freq[j] + (double)inv_freq[half + j];
          double ang = (double)positions[t] * f;
          ang -= 6.283185307179586476925286766559 * rint(ang * 0.15915494309189533576888376337251);
          float sn, cs;
          sincosf((float)ang, &sn, &cs);
          sn *= magnitude;
          cs *= magnitude;
          const float ru = u * cs - v * sn, rv = v * cs + u * sn;
          u = ru;
          v = rv;
        }
      }
    }
    *reinterpret_cast<__nv_bfloat162*>(Qs + (size_t)r * DP + d) = __floats2bfloat162_rn(u, v);
  }
  if (tid < BM) {
    row_m[tid] = -INFINITY;
    row_l[tid] = 0.f;
  }

  const int chunks = D / 8;                       // 16-byte pieces of an entry
  auto load_tile = [&](int tile, int buf) {
    __nv_bfloat16* dst = Ks + (size_t)buf * BN * DP;
    for (int c = tid; c < BN * chunks; c += THREADS) {
      const int k = c / chunks, part = c - k * chunks;
      const int key = tile * BN + k;
      bool valid = key <= max_pos;
      const __nv_bfloat16* src = cache;
      if (valid) {
        const int page = table[key / page_size];
        valid = bspec::in_range(page, n_pages, 112);
        if (valid) src = cache + ((size_t)page * page_size + key % page_size) * D + part * 8;
      }
      cp_async16(dst + (size_t)k * DP + part * 8, src, valid);
    }
  };

  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const int ntw = R / 16;                         // n-tiles this warp owns
  const int col0 = ch * (R / 2);                  // its first output column
  const int mat = lane >> 3, r8 = lane & 7;
  const int qrow = lane >> 2, qcol = 2 * (lane & 3);

  if (t_begin < t_end) load_tile(t_begin, 0);
  cp_async_commit();
  for (int tile = t_begin; tile < t_end; ++tile) {
    const int buf = (tile - t_begin) & 1;
    if (tile + 1 < t_end) load_tile(tile + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const __nv_bfloat16* Kt = Ks + (size_t)buf * BN * DP;
    // ---- S: this warp's 16 rows x 16 keys
    {
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t a[4], b[4];
        ldsm_x4(a, Qs + (size_t)(16 * rg + 8 * (mat & 1) + r8) * DP + 16 * ks + 8 * (mat >> 1));
        ldsm_x4(b, Kt + (size_t)(16 * ch + 8 * (mat >> 1) + r8) * DP + 16 * ks + 8 * (mat & 1));
        mma_bf16(s[0], a, b[0], b[1]);
        mma_bf16(s[1], a, b[2], b[3]);
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int r = 16 * rg + qrow + 8 * half;
          const long long row = row0 + r;
          const int pos = pos0 + (int)min((long long)q_len - 1, row / H);
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int c = 16 * ch + 8 * nt + qcol + j;
            const int key = tile * BN + c;
            Ss[r * SP + c] = (row < rows_total && key <= pos) ? s[nt][2 * half + j] * scale : -INFINITY;
          }
        }
    }
    __syncthreads();
    // ---- softmax: four threads per row, eight keys each
    {
      const int r = tid >> 2, part = tid & 3;
      float v[8];
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[j] = Ss[r * SP + 8 * part + j];
        mx = fmaxf(mx, v[j]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_old = row_m[r], l_old = row_l[r];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float p = m_new == -INFINITY ? 0.f : expf(v[j] - m_new);
        sum += p;
        const __nv_bfloat16 hi = __float2bfloat16_rn(p);
        Ph[r * PP + 8 * part + j] = hi;
        Pl[r * PP + 8 * part + j] = __float2bfloat16_rn(p - __bfloat162float(hi));
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      if (part == 0) {
        const float corr = m_new == -INFINITY ? 1.f : expf(m_old - m_new);
        row_m[r] = m_new;
        row_l[r] = l_old * corr + sum;
        row_c[r] = corr;
      }
    }
    __syncthreads();
    // ---- O = O * corr + P V over this warp's columns
    {
      const float c_lo = row_c[16 * rg + qrow], c_hi = row_c[16 * rg + qrow + 8];
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        o[i][0] *= c_lo; o[i][1] *= c_lo; o[i][2] *= c_hi; o[i][3] *= c_hi;
      }
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {
        uint32_t ah[4], al[4];
        ldsm_x4(ah, Ph + (size_t)(16 * rg + 8 * (mat & 1) + r8) * PP + 16 * kk + 8 * (mat >> 1));
        ldsm_x4(al, Pl + (size_t)(16 * rg + 8 * (mat & 1) + r8) * PP + 16 * kk + 8 * (mat >> 1));
#pragma unroll
        for (int nd = 0; nd < NT; nd += 2) {
          if (nd < ntw) {
            uint32_t b[4];
            ldsm_x4_trans(b, Kt + (size_t)(16 * kk + 8 * (mat & 1) + r8) * DP + col0 + 8 * (nd + (mat >> 1)));
            mma_bf16(o[nd], ah, b[0], b[1]);
            mma_bf16(o[nd], al, b[0], b[1]);
            if (nd + 1 < ntw) {
              mma_bf16(o[nd + 1], ah, b[2], b[3]);
              mma_bf16(o[nd + 1], al, b[2], b[3]);
            }
          }
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();          // row_m / row_l of the init (no tiles) or of the last tile, for every warp

  // ---- results
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = 16 * rg + qrow + 8 * half;
    const long long row = row0 + r;
    if (row >= rows_total) continue;
    const long long t = q_begin + row / H;
    const int h = (int)(row % H);
    if (n_splits == 1) {
      const float inv = 1.f / row_l[r];
      __nv_bfloat16* op = out + t * o_row + h * o_head;
#pragma unroll
      for (int nd = 0; nd < NT; ++nd)
        if (nd < ntw) {
          const int c = col0 + 8 * nd + qcol;
          *reinterpret_cast<__nv_bfloat162*>(op + c) =
              __floats2bfloat162_rn(o[nd][2 * half] * inv, o[nd][2 * half + 1] * inv);
        }
    } else {
      const size_t slot = ((size_t)t * H + h) * n_splits + split;
      float* op = o_part + slot * R;
#pragma unroll
      for (int nd = 0; nd < NT; ++nd)
        if (nd < ntw) {
          const int c = col0 + 8 * nd + qcol;
          *reinterpret_cast<float2*>(op + c) = make_float2(o[nd][2 * half], o[nd][2 * half + 1]);
        }
      if (ch == 0 && (lane & 3) == 0) {
        ml_part[2 * slot] = row_m[r];
        ml_part[2 * slot + 1] = row_l[r];
      }
    }
  }
}

// out[row, :] = sum_s w_s O_s / sum_s w_s l_s with w_s = exp(m_s - max m), s ascending.  One block per (token, head).
__global__ void latent_attn_join_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part,
                                        __nv_bfloat16* __restrict__ out, long long o_row, long long o_head, int H,
                                        int R, int n_splits) {
  bspec::pdl_prologue(44);
  const size_t row = blockIdx.x;
  const long long t = row / H;
  const int h = (int)(row % H);
  float M = -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, ml_part[2 * (row * n_splits + s)]);
  float L = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float m = ml_part[2 * (row * n_splits + s)];
    if (m != -INFINITY) L += expf(m - M) * ml_part[2 * (row * n_splits + s) + 1];
  }
  const float inv = 1.f / L;
  for (int c = threadIdx.x; c < R; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float m = ml_part[2 * (row * n_splits + s)];
      if (m != -INFINITY) acc += expf(m - M) * o_part[(row * n_splits + s) * R + c];
    }
    out[t * o_row + h * o_head + c] = __float2bfloat16_rn(acc * inv);
  }
}

}  // namespace

// 1 if the tensor-core kernel takes these sizes (ranks and rotated part multiples of 16, latent at most 512,
// the tile fits shared memory), else 0.
BSPEC_API int bspec_latent_attention_mma_supported(int R, int P) {
  return (R > 0 && R % 16 == 0 && P >= 16 && P % 16 == 0 && R <= 512 && smem_bytes(R + P) <= 220 * 1024) ? 1 : 0;
}

BSPEC_API int bspec_latent_attention_mma(const void* ql, long long ql_row, long long ql_head, const void* qr,
                                         long long qr_row, long long qr_head, void* out, long long o_row,
                                         long long o_head, const void* cache, const int* qo_indptr,
                                         const int* positions, const int* kv_indptr, const int* kv_indices,
                                         int n_entries, int n_tokens, int max_q_len, int H, int R, int P,
                                         int page_size, float scale, int n_splits, float* o_part, float* ml_part,
                                         long long n_pages, const float* inv_freq, float magnitude,
                                         cudaStream_t stream) {
  if (n_entries <= 0 || max_q_len <= 0) return 0;
  if (!bspec_latent_attention_mma_supported(R, P) || n_splits < 1 || (n_splits > 1 && (!o_part || !ml_part)))
    return (int)cudaErrorInvalidValue;
  const long long row_tiles = ((long long)max_q_len * H + BM - 1) / BM;
  if (row_tiles > 2147483647ll || n_entries > 65535 || n_splits > 65535) return (int)cudaErrorInvalidConfiguration;
  dim3 grid((unsigned)row_tiles, n_entries, n_splits);
  const size_t smem = smem_bytes(R + P);
  const int ntw = R / 16;
#define LM(N)                                                                                                        \
  do {                                                                                                               \
    cudaFuncSetAttribute(latent_attn_mma_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
    BSPEC_LAUNCH((latent_attn_mma_kernel<N>), grid, THREADS, smem, stream, (const __nv_bfloat16*)ql, ql_row, ql_head, \
                 (const __nv_bfloat16*)qr, qr_row, qr_head, (__nv_bfloat16*)out, o_row, o_head,                      \
                 (const __nv_bfloat16*)cache, qo_indptr, positions, kv_indptr, kv_indices, H, R, P, page_size,       \
                 scale, n_splits, o_part, ml_part, n_pages, inv_freq, magnitude);                                    \
  } while (0)
  if (ntw <= 8) LM(8); else if (ntw <= 16) LM(16); else LM(32);
#undef LM
  int err = BSPEC_LAUNCH_CHECK();
  if (err != 0 || n_splits == 1) return err;
  BSPEC_LAUNCH((latent_attn_join_kernel), (unsigned)((long long)n_tokens * H), R >= 256 ? 128 : 64, 0, stream, o_part,
               ml_part, (__nv_bfloat16*)out, o_row, o_head, H, R, n_splits);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_DEFINE_TRACE_SETTER(bspec_trace_set_latent_mma)
BSPEC_DEFINE_BOUNDS_REPORT(bspec_bounds_report_latent_mma)
