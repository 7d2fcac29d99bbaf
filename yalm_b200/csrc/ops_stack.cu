// Row-batched ops of the layered executor (stack.cpp): every op takes M rows = M consecutive positions of one sequence,
// M = 1 being a decode step and M > 1 a portion of a prompt, so that both run the same arithmetic.  The residual stream,
// norms, scores, softmax weights and router are fp32 whatever the weight type; weights are fp32 / fp16 / bf16 (out, in)
// row-major and every product accumulates in fp32.
//
// Mechanisms (each with its constants as parameters, so another layered design can use them):
//   embed_rows            x = E[token] (+ learned position row)
//   linear_rows           y = alpha * x W^T: warp-per-output GEMV for few rows, 64 x 64 SIMT tiles for many (the tensor-core
//                         route for 16-bit weights is prefill_gemm.cu; this is the exact-fp32 and odd-shape route)
//   qkv_post_rows         RMS norm over the whole q / k projection, value blending with an earlier layer's values, append
//                         to the key / value ring
//   kv_pool_rows          mean key / value of every token block completed by these rows
//   attn_window_pool      sliding window + pooled blocks in one softmax
//   norm_residual_rows    x += rms(sum of partial outputs) * (offset + w)
//   glu_act_rows          gated activation with clamps and up offset
//   router_topk_rows      fp32 router, sigmoid / softmax scores, top-k
//   moe_glu_slots / moe_down_slots   per (row, selected expert) projections through stacked expert matrices
//   norm_gather_rows      final norm of the rows whose logits are wanted
// Positions: p0 + row, p0 = ctl[CTL_POS] when a device control block is given (device-side decode loops), else the argument.
#include "common.cuh"

#include <cuda_bf16.h>

#include <algorithm>

#include "gemv.cuh"
#include "launch.h"
#include "stack_rows.cuh"

namespace yalm {
namespace stack {

// ---- embedding ---------------------------------------------------------------------------------------------------------
template <int DT>
__global__ void embed_rows_kernel(float *__restrict__ x, const void *__restrict__ table, const void *__restrict__ positions,
                                  const int *__restrict__ tokens, int dim, int pos0, const int *__restrict__ ctl, float scale) {
	const int m = blockIdx.x;
	const int tok = tokens ? tokens[m] : ctl[CTL_TOKEN];
	const int p = first_pos(ctl, pos0) + m;
	for (int e = threadIdx.x; e < dim; e += blockDim.x) {
		float v = Elem<DT>::get(table, (size_t)tok * dim + e) * scale;
		if (positions) v += Elem<DT>::get(positions, (size_t)p * dim + e);
		x[(size_t)m * dim + e] = v;
	}
}

// ---- linear: few rows ------------------------------------------------------------------------------------------------
// One warp per output column n, MB rows of x per pass (grid.y walks the passes): the weight row is read once per pass.
constexpr int kLinMB = 8;
template <int DT>
__global__ void __launch_bounds__(256) linear_few_kernel(float *__restrict__ y, int ldy, const float *__restrict__ x, int ldx,
                                                         const void *__restrict__ w, int M, int N, int K, float alpha, bool vec) {
	using E = Elem<DT>;
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int n = blockIdx.x * 8 + warp;
	if (n >= N) return;
	const int m0 = blockIdx.y * kLinMB, mb = min(kLinMB, M - m0);
	float acc[kLinMB];
#pragma unroll
	for (int i = 0; i < kLinMB; ++i) acc[i] = 0.f;
	const size_t row_off = (size_t)n * K;
	if (vec) {
		const typename E::T *row = static_cast<const typename E::T *>(w) + row_off;
		for (int k = lane * E::VEC; k < K; k += 32 * E::VEC) {
			float f[8];
			E::unpack(ldg_stream(row + k), f);
#pragma unroll
			for (int i = 0; i < kLinMB; ++i)
				if (i < mb) {
					const float *xr = x + (size_t)(m0 + i) * ldx + k;
#pragma unroll
					for (int j = 0; j < E::VEC; j += 4) {
						const float4 xv = *reinterpret_cast<const float4 *>(xr + j);
						acc[i] = fmaf(f[j], xv.x, acc[i]), acc[i] = fmaf(f[j + 1], xv.y, acc[i]);
						acc[i] = fmaf(f[j + 2], xv.z, acc[i]), acc[i] = fmaf(f[j + 3], xv.w, acc[i]);
					}
				}
		}
	} else {
		for (int k = lane; k < K; k += 32) {
			const float wv = E::get(w, row_off + k);
#pragma unroll
			for (int i = 0; i < kLinMB; ++i)
				if (i < mb) acc[i] = fmaf(wv, x[(size_t)(m0 + i) * ldx + k], acc[i]);
		}
	}
#pragma unroll
	for (int i = 0; i < kLinMB; ++i) {
		const float s = warp_sum(acc[i]);
		if (i < mb && lane == 0) y[(size_t)(m0 + i) * ldy + n] = alpha * s;
	}
}

// ---- linear: many rows, SIMT tiles -----------------------------------------------------------------------------------
// 64 x 64 output tile per CTA, K in steps of 16, 256 threads x (4 x 4) outputs.  Operands are staged transposed
// ([k][row]) so that the inner product reads float4s; edges are zero-filled.  fp32 multiply-add throughout: this is the
// route of the exact-fp32 mode and of shapes the tensor-core GEMM's 16-byte row rule excludes.
template <int DT>
__global__ void __launch_bounds__(256) linear_tiled_kernel(float *__restrict__ y, int ldy, const float *__restrict__ x, int ldx,
                                                           const void *__restrict__ w, int M, int N, int K, float alpha) {
	using E = Elem<DT>;
	__shared__ __align__(16) float As[16][64 + 4], Ws[16][64 + 4];
	const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
	const int tid = threadIdx.x, tm = tid >> 4, tn = tid & 15;
	const int lr = tid >> 2, lk = (tid & 3) * 4; // this thread stages row lr, k offsets lk .. lk + 3 of both operands
	float acc[4][4];
#pragma unroll
	for (int i = 0; i < 4; ++i)
#pragma unroll
		for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
	for (int k0 = 0; k0 < K; k0 += 16) {
		float a[4], b[4];
#pragma unroll
		for (int i = 0; i < 4; ++i) {
			const int k = k0 + lk + i;
			a[i] = (m0 + lr < M && k < K) ? x[(size_t)(m0 + lr) * ldx + k] : 0.f;
			b[i] = (n0 + lr < N && k < K) ? E::get(w, (size_t)(n0 + lr) * K + k) : 0.f;
		}
		__syncthreads(); // the previous step's reads are done
#pragma unroll
		for (int i = 0; i < 4; ++i) As[lk + i][lr] = a[i], Ws[lk + i][lr] = b[i];
		__syncthreads();
#pragma unroll
		for (int k = 0; k < 16; ++k) {
			const float4 av = *reinterpret_cast<const float4 *>(&As[k][tm * 4]), bv = *reinterpret_cast<const float4 *>(&Ws[k][tn * 4]);
			const float aa[4] = {av.x, av.y, av.z, av.w}, bb[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
			for (int i = 0; i < 4; ++i)
#pragma unroll
				for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(aa[i], bb[j], acc[i][j]);
		}
	}
#pragma unroll
	for (int i = 0; i < 4; ++i) {
		const int m = m0 + tm * 4 + i;
		if (m >= M) continue;
#pragma unroll
		for (int j = 0; j < 4; ++j) {
			const int n = n0 + tn * 4 + j;
			if (n < N) y[(size_t)m * ldy + n] = alpha * acc[i][j];
		}
	}
}

// fp32 rows -> 16-bit rows (the A operand of the tensor-core GEMM), K padded columns are not written
template <typename T>
__global__ void cast_rows_kernel(T *__restrict__ out, const float *__restrict__ x, int ldx, int K) {
	const float *row = x + (size_t)blockIdx.x * ldx;
	T *dst = out + (size_t)blockIdx.x * K;
	for (int e = threadIdx.x; e < K; e += blockDim.x) dst[e] = T(row[e]);
}

// ---- q / k norm, value blending, cache append ---------------------------------------------------------------------------
// Row m of qkv (fp32, q | k | v, ld) is position p0 + m.  q and k: RMS norm over the WHOLE projection (all heads at once),
// one weight per channel (qnorm / knorm null: left as they are); q stays in place, k goes to the ring.  v: vmode 1 keeps a
// copy in vfirst (the first blending layer), vmode 2 blends v = (1 - lambda) v + lambda vfirst (later blending layers);
// the blended v is what is cached.  Ring slot of position p: p % ring; caches are head-major (kv head, slot, channel).
template <typename CT>
__global__ void __launch_bounds__(256) qkv_post_rows_kernel(float *__restrict__ qkv, int ld, CT *__restrict__ kc, CT *__restrict__ vc,
                                                            float *__restrict__ vfirst, int ldvf, const float *__restrict__ qnorm,
                                                            const float *__restrict__ knorm, const float *__restrict__ vmix, int vmode, int nq,
                                                            int nk, int nv, int dk, int dv, int ring, float eps, int pos0,
                                                            const int *__restrict__ ctl) {
	__shared__ float red[33];
	const int m = blockIdx.x, p = first_pos(ctl, pos0) + m;
	qkv_post_row<CT>(qkv + (size_t)m * ld, kc, vc, vfirst ? vfirst + (size_t)m * ldvf : nullptr, qnorm, knorm, vmix, vmode, nq, nk, nv, dk, dv, ring, p % ring,
	                 eps, red);
}

// Mean key / value (fp32) of every block of `pool` positions whose last position is one of these rows; the members are read
// back from the ring, as it holds them.  grid (n / pool + 1, kv heads).
template <typename CT>
__global__ void kv_pool_rows_kernel(float *__restrict__ kp, float *__restrict__ vp, const CT *__restrict__ kc, const CT *__restrict__ vc, int n,
                                    int dk, int dv, int ring, int pool, int max_blocks, int pos0, const int *__restrict__ ctl) {
	const int p0 = first_pos(ctl, pos0);
	const int b = p0 / pool + blockIdx.x; // first block whose end (b * pool + pool - 1) is >= p0
	if (b * pool + pool > p0 + n || b >= max_blocks) return;
	kv_pool_block<CT>(kp, vp, kc, vc, b, blockIdx.y, dk, dv, ring, pool, max_blocks);
}

// ---- attention: sliding window + pooled blocks, one softmax ------------------------------------------------------------
// Query row m at position i = p0 + m sees the tokens lo .. i (lo = max(0, i - window + 1); window 0: lo = 0) and, when
// pool > 0, the blocks 0 .. nb - 1 with nb = floor((i - window + 1) / pool): those whose last token has left the window.
// One CTA per (kv head x group of up to R query heads that share it, row, split): the key / value rows are read once for
// the R heads.  Its warps take 32-key tiles in turn: lane = key for the scores (each lane walks its own key row against
// the R queries in shared memory), online softmax per warp and head in fp32, then lane = value channel for P V.  Warps
// merge in shared memory; with more than one split (few rows: decoding) the CTA leaves an unnormalised partial
// (accumulator, max, sum) and attn_merge_kernel combines the splits in order.
constexpr int kAttnWarps = 4;
constexpr int kAttnMaxParts = 4096; // (row, head, split) partials the workspace holds

template <typename CT, int R>
__device__ __forceinline__ void key_dots(const CT *krow, const float *qs, int dkp, int dk, bool vec, float (&s)[R]);
template <int R>
__device__ __forceinline__ void key_dots_f32(const float *krow, const float *qs, int dkp, int dk, bool vec, float (&s)[R]) {
	if (vec) {
		for (int d = 0; d < dk; d += 4) {
			const float4 kv = *reinterpret_cast<const float4 *>(krow + d);
#pragma unroll
			for (int r = 0; r < R; ++r) {
				const float4 qv = *reinterpret_cast<const float4 *>(qs + r * dkp + d);
				s[r] = fmaf(kv.x, qv.x, s[r]), s[r] = fmaf(kv.y, qv.y, s[r]), s[r] = fmaf(kv.z, qv.z, s[r]), s[r] = fmaf(kv.w, qv.w, s[r]);
			}
		}
	} else
		for (int d = 0; d < dk; ++d) {
			const float kv = krow[d];
#pragma unroll
			for (int r = 0; r < R; ++r) s[r] = fmaf(kv, qs[r * dkp + d], s[r]);
		}
}
template <int R>
__device__ __forceinline__ void key_dots_bf16(const __nv_bfloat16 *krow, const float *qs, int dkp, int dk, bool vec, float (&s)[R]) {
	if (vec && dk % 64 == 0) { // eight 16-byte pieces of the row in flight per lane: one memory round trip per 64 channels
		for (int d0 = 0; d0 < dk; d0 += 64) {
			uint4 w[8];
#pragma unroll
			for (int j = 0; j < 8; ++j) w[j] = __ldg(reinterpret_cast<const uint4 *>(krow + d0 + 8 * j));
#pragma unroll
			for (int j = 0; j < 8; ++j) {
				float f[8];
				Elem<YALM_BF16>::unpack(w[j], f);
				const int d = d0 + 8 * j;
#pragma unroll
				for (int r = 0; r < R; ++r) {
					const float4 q0 = *reinterpret_cast<const float4 *>(qs + r * dkp + d), q1 = *reinterpret_cast<const float4 *>(qs + r * dkp + d + 4);
					s[r] = fmaf(f[0], q0.x, s[r]), s[r] = fmaf(f[1], q0.y, s[r]), s[r] = fmaf(f[2], q0.z, s[r]), s[r] = fmaf(f[3], q0.w, s[r]);
					s[r] = fmaf(f[4], q1.x, s[r]), s[r] = fmaf(f[5], q1.y, s[r]), s[r] = fmaf(f[6], q1.z, s[r]), s[r] = fmaf(f[7], q1.w, s[r]);
				}
			}
		}
	} else if (vec) {
		for (int d = 0; d < dk; d += 8) {
			float f[8];
			Elem<YALM_BF16>::unpack(*reinterpret_cast<const uint4 *>(krow + d), f);
#pragma unroll
			for (int r = 0; r < R; ++r) {
				const float4 q0 = *reinterpret_cast<const float4 *>(qs + r * dkp + d), q1 = *reinterpret_cast<const float4 *>(qs + r * dkp + d + 4);
				s[r] = fmaf(f[0], q0.x, s[r]), s[r] = fmaf(f[1], q0.y, s[r]), s[r] = fmaf(f[2], q0.z, s[r]), s[r] = fmaf(f[3], q0.w, s[r]);
				s[r] = fmaf(f[4], q1.x, s[r]), s[r] = fmaf(f[5], q1.y, s[r]), s[r] = fmaf(f[6], q1.z, s[r]), s[r] = fmaf(f[7], q1.w, s[r]);
			}
		}
	} else
		for (int d = 0; d < dk; ++d) {
			const float kv = cache_get(krow, d);
#pragma unroll
			for (int r = 0; r < R; ++r) s[r] = fmaf(kv, qs[r * dkp + d], s[r]);
		}
}
template <int R> __device__ __forceinline__ void key_dots_any(const float *krow, const float *qs, int dkp, int dk, bool vec, float (&s)[R]) {
	key_dots_f32<R>(krow, qs, dkp, dk, vec, s);
}
template <int R> __device__ __forceinline__ void key_dots_any(const __nv_bfloat16 *krow, const float *qs, int dkp, int dk, bool vec, float (&s)[R]) {
	key_dots_bf16<R>(krow, qs, dkp, dk, vec, s);
}

template <typename CT, int R, int DVC>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_window_pool_kernel(float *__restrict__ out, int ldo, const float *__restrict__ q, int ldq,
                                                                           const CT *__restrict__ kc, const CT *__restrict__ vc,
                                                                           const float *__restrict__ kp, const float *__restrict__ vp,
                                                                           float *__restrict__ part, int n_heads, int n_kv, int dk, int dv, int ring,
                                                                           int max_blocks, int window, int pool, float scale, int pos0,
                                                                           const int *__restrict__ ctl, int ldk, int ldv, const float *__restrict__ sink,
                                                                           int v_heads) {
	extern __shared__ __align__(16) float sm[];
	const int dkp = (dk + 7) & ~7;
	float *qs = sm;                                    // R x dkp
	float *macc = qs + R * dkp;                        // kAttnWarps x R x dv
	float *mml = macc + kAttnWarps * R * dv;           // kAttnWarps x R x 2
	const int rep = n_heads / n_kv, hg = (rep + R - 1) / R;
	const int g = blockIdx.x / hg, h0 = g * rep + (blockIdx.x % hg) * R, nh = min(R, g * rep + rep - h0);
	const int m = blockIdx.y, z = blockIdx.z, nsplit = gridDim.z;
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int i = first_pos(ctl, pos0) + m;
	const int lo = window > 0 ? max(0, i - window + 1) : 0;
	const int nb = (window > 0 && pool > 0 && i - window + 1 >= pool) ? min((i - window + 1) / pool, max_blocks) : 0; // the pooled buffers hold max_blocks
	for (int e = threadIdx.x; e < R * dkp; e += blockDim.x) {
		const int r = e / dkp, d = e % dkp;
		qs[e] = (r < nh && d < dk) ? q[(size_t)m * ldq + (size_t)(h0 + r) * dk + d] * scale : 0.f;
	}
	__syncthreads();
	const int gv = g % v_heads; // key heads beyond the value heads (further maps over the same values) wrap around
	const CT *kbase = kc + (size_t)g * ring * ldk, *vbase = vc + (size_t)gv * ring * ldv; // ldk, ldv: row strides of the rings (dk, dv when packed)
	const float *kpb = kp ? kp + (size_t)g * max_blocks * dk : nullptr, *vpb = vp ? vp + (size_t)gv * max_blocks * dv : nullptr;
	const bool kvec_c = (dk * sizeof(CT)) % 16 == 0 && (ldk * sizeof(CT)) % 16 == 0 && aligned16(kbase), kvec_p = (dk * 4) % 16 == 0 && aligned16(kpb);
	float mx[R], l[R], acc[R][DVC];
#pragma unroll
	for (int r = 0; r < R; ++r) {
		mx[r] = -INFINITY, l[r] = 0.f;
#pragma unroll
		for (int c = 0; c < DVC; ++c) acc[r][c] = 0.f;
	}
	// pooled blocks and tokens occupy separate 32-key tiles, so that a tile's rows are of one kind (fp32 means or cache rows)
	const int ntok = i - lo + 1, ptiles = (nb + 31) / 32, ntiles = ptiles + (ntok + 31) / 32, per = (ntiles + nsplit - 1) / nsplit;
	const int t_end = min(ntiles, (z + 1) * per);
	for (int t = z * per + warp; t < t_end; t += kAttnWarps) {
		const bool pooled = t < ptiles;
		const int idx0 = pooled ? t * 32 : (t - ptiles) * 32, cnt = min(32, (pooled ? nb : ntok) - idx0);
		float s[R], p[R];
#pragma unroll
		for (int r = 0; r < R; ++r) s[r] = 0.f;
		if (lane < cnt) {
			if (pooled) key_dots_f32<R>(kpb + (size_t)(idx0 + lane) * dk, qs, dkp, dk, kvec_p, s);
			else key_dots_any<R>(kbase + (size_t)((lo + idx0 + lane) % ring) * ldk, qs, dkp, dk, kvec_c, s);
		}
#pragma unroll
		for (int r = 0; r < R; ++r) {
			const float sv = lane < cnt ? s[r] : -INFINITY;
			const float nmx = fmaxf(mx[r], warp_max(sv));     // finite: the tile holds at least one key
			const float corr = mx[r] == -INFINITY ? 0.f : expf(mx[r] - nmx);
			p[r] = lane < cnt ? expf(sv - nmx) : 0.f;
			l[r] = l[r] * corr + warp_sum(p[r]);
			mx[r] = nmx;
#pragma unroll
			for (int c = 0; c < DVC; ++c) acc[r][c] *= corr;
		}
		// P V: lane = value channel; the value rows of KU keys are fetched before the first multiply (one L2 round trip per KU keys)
		constexpr int KU = 8;
		for (int k0 = 0; k0 < cnt; k0 += KU) {
			float vv[KU][DVC];
#pragma unroll
			for (int j = 0; j < KU; ++j) {
				const int kk = min(k0 + j, cnt - 1); // past the end: a repeated row whose weight is zero
				if (pooled) {
					const float *vr = vpb + (size_t)(idx0 + kk) * dv;
#pragma unroll
					for (int c = 0; c < DVC; ++c) vv[j][c] = c * 32 + lane < dv ? vr[c * 32 + lane] : 0.f;
				} else {
					const CT *vr = vbase + (size_t)((lo + idx0 + kk) % ring) * ldv;
#pragma unroll
					for (int c = 0; c < DVC; ++c) vv[j][c] = c * 32 + lane < dv ? cache_get(vr, c * 32 + lane) : 0.f;
				}
			}
#pragma unroll
			for (int j = 0; j < KU; ++j)
#pragma unroll
				for (int r = 0; r < R; ++r) {
					const float pk = k0 + j < cnt ? __shfl_sync(kFull, p[r], (k0 + j) & 31) : 0.f;
#pragma unroll
					for (int c = 0; c < DVC; ++c) acc[r][c] = fmaf(pk, vv[j][c], acc[r][c]);
				}
		}
	}
#pragma unroll
	for (int r = 0; r < R; ++r) {
#pragma unroll
		for (int c = 0; c < DVC; ++c)
			if (c * 32 + lane < dv) macc[(warp * R + r) * dv + c * 32 + lane] = acc[r][c];
		if (lane == 0) mml[(warp * R + r) * 2] = mx[r], mml[(warp * R + r) * 2 + 1] = l[r];
	}
	__syncthreads();
	for (int r = warp; r < nh; r += kAttnWarps) { // one warp finishes one head
		float M = -INFINITY;
		for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, mml[(w * R + r) * 2]);
		float wt[kAttnWarps], L = 0.f;
		for (int w = 0; w < kAttnWarps; ++w) {
			const float mw = mml[(w * R + r) * 2];
			wt[w] = mw == -INFINITY ? 0.f : expf(mw - M);
			L += wt[w] * mml[(w * R + r) * 2 + 1];
		}
		const int h = h0 + r;
		float *pr = part ? part + ((size_t)(m * n_heads + h) * nsplit + z) * (dv + 2) : nullptr;
		for (int c = lane; c < dv; c += 32) {
			float o = 0.f;
			for (int w = 0; w < kAttnWarps; ++w) o += wt[w] * macc[(w * R + r) * dv + c];
			if (pr) pr[c] = o;
			else out[(size_t)m * ldo + (size_t)h * dv + c] = o * softmax_finish(M, L, sink, h);
		}
		if (pr && lane == 0) pr[dv] = M, pr[dv + 1] = L;
	}
}

// The same attention for bf16 rings whose key and value sizes are 8, 16, ..., 256: every row is read as 16-byte pieces by
// dk / 8 (dv / 8) neighbouring lanes, so that one warp instruction fetches whole rows and eight of them are in flight per
// lane; each lane keeps its 8 channels of the R queries and of the R accumulators in registers.  Scores of a 32-key tile
// pass through shared memory between the two phases (lane = key for the softmax bookkeeping).  Block means (fp32) are read
// in the same lane layout as two 16-byte pieces.  Same grid, splits, partials and merge as attn_window_pool_kernel.
template <int R>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_window_pool_lanes_kernel(float *__restrict__ out, int ldo, const float *__restrict__ q, int ldq,
                                                                                 const __nv_bfloat16 *__restrict__ kc,
                                                                                 const __nv_bfloat16 *__restrict__ vc, const float *__restrict__ kp,
                                                                                 const float *__restrict__ vp, float *__restrict__ part, int n_heads,
                                                                                 int n_kv, int dk, int dv, int ring, int max_blocks, int window, int pool,
                                                                                 float scale, int pos0, const int *__restrict__ ctl,
                                                                                 const float *__restrict__ sink, int v_heads) {
	extern __shared__ __align__(16) float sm[];
	float *qs = sm;                                    // R x dk
	float *macc = qs + R * dk;                         // kAttnWarps x R x dv
	float *mml = macc + kAttnWarps * R * dv;           // kAttnWarps x R x 2
	float *sc = mml + kAttnWarps * R * 2;              // kAttnWarps x R x 32
	const int rep = n_heads / n_kv, hg = (rep + R - 1) / R;
	const int g = blockIdx.x / hg, h0 = g * rep + (blockIdx.x % hg) * R, nh = min(R, g * rep + rep - h0);
	const int m = blockIdx.y, z = blockIdx.z, nsplit = gridDim.z;
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int i = first_pos(ctl, pos0) + m;
	const int lo = window > 0 ? max(0, i - window + 1) : 0;
	const int nb = (window > 0 && pool > 0 && i - window + 1 >= pool) ? min((i - window + 1) / pool, max_blocks) : 0; // the pooled buffers hold max_blocks
	for (int e = threadIdx.x; e < R * dk; e += blockDim.x) {
		const int r = e / dk, d = e % dk;
		qs[e] = r < nh ? q[(size_t)m * ldq + (size_t)(h0 + r) * dk + d] * scale : 0.f;
	}
	__syncthreads();
	const int LK = dk >> 3, LV = dv >> 3;                          // lanes per key / value row
	const int subk = lane % LK, rgk = lane / LK, rpk = 32 / LK;    // piece of the row, row within a step, rows per step
	const int subv = lane % LV, rgv = lane / LV, rpv = 32 / LV;
	float qr[R][8];
#pragma unroll
	for (int r = 0; r < R; ++r)
#pragma unroll
		for (int j = 0; j < 8; ++j) qr[r][j] = qs[r * dk + subk * 8 + j];
	const int gv = g % v_heads; // key heads beyond the value heads (further maps over the same values) wrap around
	const __nv_bfloat16 *kbase = kc + (size_t)g * ring * dk + subk * 8, *vbase = vc + (size_t)gv * ring * dv + subv * 8;
	const float *kpb = kp ? kp + (size_t)g * max_blocks * dk + subk * 8 : nullptr, *vpb = vp ? vp + (size_t)gv * max_blocks * dv + subv * 8 : nullptr;
	float *scw = sc + warp * R * 32;
	float mx[R], l[R], acc[R][8];
#pragma unroll
	for (int r = 0; r < R; ++r) {
		mx[r] = -INFINITY, l[r] = 0.f;
#pragma unroll
		for (int j = 0; j < 8; ++j) acc[r][j] = 0.f;
	}
	const int ntok = i - lo + 1, ptiles = (nb + 31) / 32, ntiles = ptiles + (ntok + 31) / 32, per = (ntiles + nsplit - 1) / nsplit;
	const int t_end = min(ntiles, (z + 1) * per);
	constexpr int KU = 8; // row steps in flight
	for (int t = z * per + warp; t < t_end; t += kAttnWarps) {
		const bool pooled = t < ptiles;
		const int idx0 = pooled ? t * 32 : (t - ptiles) * 32, cnt = min(32, (pooled ? nb : ntok) - idx0);
		// ---- scores ----
		for (int u0 = 0; u0 * rpk < cnt; u0 += KU) {
			float kf[KU][8];
			if (pooled) {
#pragma unroll
				for (int u = 0; u < KU; ++u) {
					const float *kr = kpb + (size_t)(idx0 + min((u0 + u) * rpk + rgk, cnt - 1)) * dk;
					const float4 a = __ldg(reinterpret_cast<const float4 *>(kr)), b = __ldg(reinterpret_cast<const float4 *>(kr + 4));
					kf[u][0] = a.x, kf[u][1] = a.y, kf[u][2] = a.z, kf[u][3] = a.w, kf[u][4] = b.x, kf[u][5] = b.y, kf[u][6] = b.z, kf[u][7] = b.w;
				}
			} else {
				uint4 w[KU];
#pragma unroll
				for (int u = 0; u < KU; ++u)
					w[u] = __ldg(reinterpret_cast<const uint4 *>(kbase + (size_t)((lo + idx0 + min((u0 + u) * rpk + rgk, cnt - 1)) % ring) * dk));
#pragma unroll
				for (int u = 0; u < KU; ++u) Elem<YALM_BF16>::unpack(w[u], kf[u]);
			}
#pragma unroll
			for (int u = 0; u < KU; ++u) {
				const int row = (u0 + u) * rpk + rgk;
				float d[R];
#pragma unroll
				for (int r = 0; r < R; ++r) {
					d[r] = 0.f;
#pragma unroll
					for (int j = 0; j < 8; ++j) d[r] = fmaf(kf[u][j], qr[r][j], d[r]);
				}
				for (int o = LK >> 1; o > 0; o >>= 1)
#pragma unroll
					for (int r = 0; r < R; ++r) d[r] += __shfl_xor_sync(kFull, d[r], o);
				if (subk == 0 && row < 32) {
#pragma unroll
					for (int r = 0; r < R; ++r) scw[r * 32 + row] = d[r];
				}
			}
		}
		__syncwarp();
		// ---- online softmax, lane = key ----
#pragma unroll
		for (int r = 0; r < R; ++r) {
			const float sv = lane < cnt ? scw[r * 32 + lane] : -INFINITY;
			const float nmx = fmaxf(mx[r], warp_max(sv)); // finite: the tile holds at least one key
			const float corr = mx[r] == -INFINITY ? 0.f : expf(mx[r] - nmx);
			const float pv = lane < cnt ? expf(sv - nmx) : 0.f;
			l[r] = l[r] * corr + warp_sum(pv);
			mx[r] = nmx;
			scw[r * 32 + lane] = pv;
#pragma unroll
			for (int j = 0; j < 8; ++j) acc[r][j] *= corr;
		}
		__syncwarp();
		// ---- P V ----
		for (int u0 = 0; u0 * rpv < cnt; u0 += KU) {
			float vf[KU][8];
			if (pooled) {
#pragma unroll
				for (int u = 0; u < KU; ++u) {
					const float *vr = vpb + (size_t)(idx0 + min((u0 + u) * rpv + rgv, cnt - 1)) * dv;
					const float4 a = __ldg(reinterpret_cast<const float4 *>(vr)), b = __ldg(reinterpret_cast<const float4 *>(vr + 4));
					vf[u][0] = a.x, vf[u][1] = a.y, vf[u][2] = a.z, vf[u][3] = a.w, vf[u][4] = b.x, vf[u][5] = b.y, vf[u][6] = b.z, vf[u][7] = b.w;
				}
			} else {
				uint4 w[KU];
#pragma unroll
				for (int u = 0; u < KU; ++u)
					w[u] = __ldg(reinterpret_cast<const uint4 *>(vbase + (size_t)((lo + idx0 + min((u0 + u) * rpv + rgv, cnt - 1)) % ring) * dv));
#pragma unroll
				for (int u = 0; u < KU; ++u) Elem<YALM_BF16>::unpack(w[u], vf[u]);
			}
#pragma unroll
			for (int u = 0; u < KU; ++u) {
				const int row = (u0 + u) * rpv + rgv;
#pragma unroll
				for (int r = 0; r < R; ++r) {
					const float pk = row < cnt ? scw[r * 32 + row] : 0.f; // past the end: a repeated row with no weight
#pragma unroll
					for (int j = 0; j < 8; ++j) acc[r][j] = fmaf(pk, vf[u][j], acc[r][j]);
				}
			}
		}
		__syncwarp(); // the next tile's scores overwrite scw
	}
	// the row groups of a warp hold partial sums of the same channels
	for (int o = 16; o >= LV; o >>= 1)
#pragma unroll
		for (int r = 0; r < R; ++r)
#pragma unroll
			for (int j = 0; j < 8; ++j) acc[r][j] += __shfl_xor_sync(kFull, acc[r][j], o);
#pragma unroll
	for (int r = 0; r < R; ++r) {
		if (rgv == 0) {
#pragma unroll
			for (int j = 0; j < 8; ++j) macc[(warp * R + r) * dv + subv * 8 + j] = acc[r][j];
		}
		if (lane == 0) mml[(warp * R + r) * 2] = mx[r], mml[(warp * R + r) * 2 + 1] = l[r];
	}
	__syncthreads();
	for (int r = warp; r < nh; r += kAttnWarps) { // one warp finishes one head
		float M = -INFINITY;
		for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, mml[(w * R + r) * 2]);
		float wt[kAttnWarps], L = 0.f;
		for (int w = 0; w < kAttnWarps; ++w) {
			const float mw = mml[(w * R + r) * 2];
			wt[w] = mw == -INFINITY ? 0.f : expf(mw - M);
			L += wt[w] * mml[(w * R + r) * 2 + 1];
		}
		const int h = h0 + r;
		float *pr = part ? part + ((size_t)(m * n_heads + h) * nsplit + z) * (dv + 2) : nullptr;
		for (int c = lane; c < dv; c += 32) {
			float o = 0.f;
			for (int w = 0; w < kAttnWarps; ++w) o += wt[w] * macc[(w * R + r) * dv + c];
			if (pr) pr[c] = o;
			else out[(size_t)m * ldo + (size_t)h * dv + c] = o * softmax_finish(M, L, sink, h);
		}
		if (pr && lane == 0) pr[dv] = M, pr[dv + 1] = L;
	}
}

// out[m, h, :] = sum_z w_z acc_z / sum_z w_z L_z with w_z = exp(M_z - max M), splits taken in order.  grid (heads, rows).
__global__ void attn_merge_kernel(float *__restrict__ out, int ldo, const float *__restrict__ part, int n_heads, int dv, int nsplit,
                                  const float *__restrict__ sink) {
	const int h = blockIdx.x, m = blockIdx.y;
	const float *pr = part + (size_t)(m * n_heads + h) * nsplit * (dv + 2);
	float M = -INFINITY;
	for (int z = 0; z < nsplit; ++z) M = fmaxf(M, pr[(size_t)z * (dv + 2) + dv]);
	float L = 0.f;
	for (int z = 0; z < nsplit; ++z) {
		const float mz = pr[(size_t)z * (dv + 2) + dv];
		if (mz != -INFINITY) L += expf(mz - M) * pr[(size_t)z * (dv + 2) + dv + 1];
	}
	const float fin = softmax_finish(M, L, sink, h);
	for (int c = threadIdx.x; c < dv; c += blockDim.x) {
		float o = 0.f;
		for (int z = 0; z < nsplit; ++z) {
			const float mz = pr[(size_t)z * (dv + 2) + dv];
			if (mz != -INFINITY) o += expf(mz - M) * pr[(size_t)z * (dv + 2) + c];
		}
		out[(size_t)m * ldo + (size_t)h * dv + c] = o * fin;
	}
}

// ---- x += rms(sum_j y_j) * (offset + w) ------------------------------------------------------------------------------------
// y holds nsum partial outputs per row (row m, part j at row m * nsum + j): the sum over a row's selected experts in slot
// order, or the single output of a dense sublayer.  The residual stream is fp32.
__global__ void __launch_bounds__(256) norm_residual_rows_kernel(float *__restrict__ x, const float *__restrict__ y, int ldy, int nsum,
                                                                 const float *__restrict__ w, float woff, float eps, int dim) {
	__shared__ float red[33];
	extern __shared__ float ys[]; // dim
	const int m = blockIdx.x;
	norm_residual_row(x + (size_t)m * dim, y + (size_t)m * nsum * ldy, ldy, nsum, w, woff, eps, dim, ys, red);
}

// out[r] = rms(x[rows[r]]) * (offset + w)   (rows null: r itself)
__global__ void __launch_bounds__(256) norm_gather_rows_kernel(float *__restrict__ out, const float *__restrict__ x, const int *__restrict__ rows,
                                                               const float *__restrict__ w, int scalar, float woff, float eps, int dim) {
	__shared__ float red[33];
	const int r = blockIdx.x, m = rows ? rows[r] : r;
	const float *src = x + (size_t)m * dim;
	float ss = 0.f;
	for (int e = threadIdx.x; e < dim; e += blockDim.x) ss += src[e] * src[e];
	ss = block_sum(ss, red);
	const float s = 1.0f / sqrtf(ss / dim + eps);
	for (int e = threadIdx.x; e < dim; e += blockDim.x) out[(size_t)r * dim + e] = src[e] * s * (woff + w[scalar ? 0 : e]);
}

// ---- gated activation ------------------------------------------------------------------------------------------------
// h[m, f] = act(gu[m, f]) * (gu[m, ff + f] + up_offset)
__global__ void glu_act_rows_kernel(float *__restrict__ h, const float *__restrict__ gu, int ff, int act, float alpha, float limit, float up_offset) {
	const int m = blockIdx.y;
	const int f = blockIdx.x * blockDim.x + threadIdx.x;
	if (f >= ff) return;
	const float *row = gu + (size_t)m * 2 * ff;
	h[(size_t)m * ff + f] = glu_value(row[f], row[ff + f], act, alpha, limit, up_offset);
}

// ---- router ----------------------------------------------------------------------------------------------------------
// z = Wr x (fp32), scores = sigmoid(z) or softmax(z); the `top` largest (ties: the lower index) with their scores as
// weights, optionally divided by their sum (+ renorm_eps).  groups > 1: the experts form `groups` equal groups of
// neighbours, a group scores its best expert, and only experts of the `keep` best groups (ties: the lower index) can be
// chosen.  One CTA per row; E <= 1024.
template <int DT>
__global__ void __launch_bounds__(256) router_topk_rows_kernel(int *__restrict__ ids, float *__restrict__ wts, const float *__restrict__ x, int ldx,
                                                               const void *__restrict__ wr, int E, int top, int dim, int score, int renorm,
                                                               float renorm_eps, int groups, int keep, bool vec, const float *__restrict__ bias,
                                                               float wscale) {
	extern __shared__ float sc[]; // E, then E logits as they were
	const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const float *xr = x + (size_t)m * ldx;
	for (int e = warp; e < E; e += (int)(blockDim.x >> 5)) {
		const float z = warp_dot<DT>(wr, (size_t)e * dim, xr, dim, vec);
		if (lane == 0) sc[e] = z;
	}
	float *ch = sc + E + groups; // E: score + bias
	if (bias)
		for (int e = threadIdx.x; e < E; e += blockDim.x) ch[e] = bias[e];
	__syncthreads();
	if (threadIdx.x == 0) {
		// The experts are ranked by their logits: both score functions are monotonic, and in fp32 a saturated sigmoid (or an
		// underflowed softmax term) would tie experts whose exact scores still differ.  Ties go to the lower index.
		float mx = -INFINITY, sum = 0.f;
		if (score != 1) {
			for (int e = 0; e < E; ++e) mx = fmaxf(mx, sc[e]);
			for (int e = 0; e < E; ++e) sum += expf(sc[e] - mx);
		}
		if (groups > 1 && keep < groups) {
			// a group's rank is its best logit; groups outside the `keep` best lose all their experts
			float *gbest = sc + E; // groups
			const int per = E / groups;
			for (int g = 0; g < groups; ++g) {
				float b = -INFINITY;
				for (int e = g * per; e < (g + 1) * per; ++e) b = fmaxf(b, sc[e]);
				gbest[g] = b;
			}
			for (int g = 0; g < groups; ++g) {
				int better = 0;
				for (int o = 0; o < groups; ++o) better += (gbest[o] > gbest[g]) || (gbest[o] == gbest[g] && o < g);
				if (better >= keep)
					for (int e = g * per; e < (g + 1) * per; ++e) sc[e] = -INFINITY;
			}
		}
		float tot = 0.f;
		if (bias) {
			// the choice adds a stored bias to the score, so it cannot be ranked by the logits: rank score + bias, weigh by the score
			for (int e = 0; e < E; ++e) {
				sc[e] = sc[e] == -INFINITY ? 0.f : (score == 1 ? 1.0f / (1.0f + expf(-sc[e])) : expf(sc[e] - mx) / sum);
				ch[e] += sc[e];
			}
			for (int j = 0; j < top; ++j) {
				int best = -1;
				float bz = -INFINITY;
				for (int e = 0; e < E; ++e)
					if (ch[e] > bz) bz = ch[e], best = e;
				if (best < 0) best = 0;
				ids[(size_t)m * top + j] = best, wts[(size_t)m * top + j] = sc[best];
				tot += sc[best];
				ch[best] = -INFINITY;
			}
		} else
		for (int j = 0; j < top; ++j) {
			int best = -1;
			float bz = -INFINITY;
			for (int e = 0; e < E; ++e)
				if (sc[e] > bz) bz = sc[e], best = e;
			if (best < 0) best = 0, bz = sc[0]; // every logit -inf or NaN: keep the indices valid
			const float bv = score == 1 ? 1.0f / (1.0f + expf(-bz)) : expf(bz - mx) / sum;
			ids[(size_t)m * top + j] = best, wts[(size_t)m * top + j] = bv;
			tot += bv;
			sc[best] = -INFINITY;
		}
		if (renorm || wscale != 1.f) { // both at once: the weights make one trip to memory and back
			const float den = renorm ? tot + renorm_eps : 1.f;
			for (int j = 0; j < top; ++j) {
				float v = wts[(size_t)m * top + j];
				if (renorm) v /= den;
				if (wscale != 1.f) v *= wscale;
				wts[(size_t)m * top + j] = v;
			}
		}
	}
}

// ---- experts, one (row, selected expert) slot at a time -------------------------------------------------------------------
// Stacked expert matrices: gate / up (E, ff, dim), down (E, dim, ff).  Slot s = row s / top, expert ids[s], weight wts[s].
// in_scale: the weight multiplies the expert's input — W (w h) = w (W h), applied to both projections before the
// activation; otherwise it multiplies the expert's output (moe_down_slots).
template <int DT>
__global__ void __launch_bounds__(128) moe_glu_slots_kernel(float *__restrict__ h, const float *__restrict__ x, int ldx, const void *__restrict__ wg,
                                                            const void *__restrict__ wu, const int *__restrict__ ids, const float *__restrict__ wts,
                                                            int top, int ff, int dim, int act, float alpha, float limit, float up_offset, int in_scale,
                                                            bool vec, int n_real) {
	const int s = blockIdx.y, f = blockIdx.x * 4 + (threadIdx.x >> 5);
	if (f >= ff) return;
	const int e = ids[s];
	if (e >= n_real) return; // an identity expert: no matrices
	const float *xr = x + (size_t)(s / top) * ldx;
	const size_t off = ((size_t)e * ff + f) * dim;
	float a = warp_dot<DT>(wg, off, xr, dim, vec), b = warp_dot<DT>(wu, off, xr, dim, vec);
	if (in_scale) a *= wts[s], b *= wts[s];
	if ((threadIdx.x & 31) == 0) h[(size_t)s * ff + f] = glu_value(a, b, act, alpha, limit, up_offset);
}
template <int DT>
__global__ void __launch_bounds__(128) moe_down_slots_kernel(float *__restrict__ y, int ldy, const float *__restrict__ h, const void *__restrict__ wd,
                                                             const int *__restrict__ ids, const float *__restrict__ wts, int ff, int dim, int out_scale,
                                                             bool vec, int n_real, const float *__restrict__ xin, int ldx, int top) {
	const int s = blockIdx.y, n = blockIdx.x * 4 + (threadIdx.x >> 5);
	if (n >= dim) return;
	const int e = ids[s];
	if (e >= n_real) { // an identity expert returns its input
		if ((threadIdx.x & 31) == 0) y[(size_t)s * ldy + n] = xin[(size_t)(s / top) * ldx + n] * (out_scale ? wts[s] : 1.f);
		return;
	}
	float v = warp_dot<DT>(wd, ((size_t)e * dim + n) * ff, h + (size_t)s * ff, ff, vec);
	if (out_scale) v *= wts[s];
	if ((threadIdx.x & 31) == 0) y[(size_t)s * ldy + n] = v;
}

// Slots of identity experts (ids >= n_real): y[s] = the slot's row of x (times its weight if out_scale).  One CTA per slot.
__global__ void moe_identity_slots_kernel(float *__restrict__ y, int ldy, const float *__restrict__ x, int ldx, const int *__restrict__ ids,
                                          const float *__restrict__ wts, int top, int dim, int n_real, int out_scale) {
	const int s = blockIdx.x;
	if (ids[s] < n_real) return;
	const float w = out_scale ? wts[s] : 1.f;
	for (int e = threadIdx.x; e < dim; e += blockDim.x) y[(size_t)s * ldy + e] = x[(size_t)(s / top) * ldx + e] * w;
}

// ---- experts, rows grouped by expert (prompt portions on the tensor cores) ---------------------------------------------------
// order[j]: the slot (row * top + k) that sits at place j once the slots are sorted by expert.  out16[j, :] = the slot's row
// of x, times the slot's weight when the weight multiplies the expert's input, rounded to the 16-bit operand type.
template <typename T>
__global__ void moe_gather_rows_kernel(T *__restrict__ out, const float *__restrict__ x, int ldx, const int *__restrict__ order,
                                       const float *__restrict__ wts, int top, int K, int in_scale) {
	const int s = order[blockIdx.x];
	const float w = in_scale ? wts[s] : 1.f;
	const float *row = x + (size_t)(s / top) * ldx;
	T *dst = out + (size_t)blockIdx.x * K;
	for (int e = threadIdx.x; e < K; e += blockDim.x) dst[e] = T(row[e] * w);
}
// y[order[j], :] = ys[j, :] (times the slot's weight when it multiplies the expert's output): back to slot order
__global__ void moe_scatter_rows_kernel(float *__restrict__ y, int ldy, const float *__restrict__ ys, int lds, const int *__restrict__ order,
                                        const float *__restrict__ wts, int dim, int out_scale) {
	const int s = order[blockIdx.x];
	const float w = out_scale ? wts[s] : 1.f;
	const float *src = ys + (size_t)blockIdx.x * lds;
	float *dst = y + (size_t)s * ldy;
	for (int e = threadIdx.x; e < dim; e += blockDim.x) dst[e] = src[e] * w;
}

} // namespace stack
} // namespace yalm

using namespace yalm;
using namespace yalm::stack;

#define DISPATCH_DT(dtype, CALL)                                                                                                   \
	switch (dtype) {                                                                                                               \
	case YALM_F32: { constexpr int DT = YALM_F32; CALL; break; }                                                                  \
	case YALM_F16: { constexpr int DT = YALM_F16; CALL; break; }                                                                  \
	case YALM_BF16: { constexpr int DT = YALM_BF16; CALL; break; }                                                                \
	default: return YALM_EINVAL;                                                                                                   \
	}

static inline int elem_size(int dtype) { return dtype == YALM_F32 ? 4 : 2; }
static inline bool row_vec(const void *w, int K, int dtype) { return aligned16(w) && ((size_t)K * elem_size(dtype)) % 16 == 0; }

extern "C" int yalm_embed_rows(float *x, const void *table, const void *positions, int dtype, const int *tokens, int n, int dim, int pos0,
                               const int *ctl, float scale, yalm_stream_t s) {
	if (!x || !table || n < 1 || dim < 1 || (!tokens && !ctl)) return YALM_EINVAL;
	DISPATCH_DT(dtype, (embed_rows_kernel<DT><<<n, 256, 0, (cudaStream_t)s>>>(x, table, positions, tokens, dim, pos0, ctl, scale)));
	return (int)cudaGetLastError();
}

// y (M, ldy) fp32 = alpha * x (M, ldx) fp32 * w (N, K)^T.  `few` rows: one warp per output column; else SIMT tiles.
extern "C" int yalm_linear_rows(float *y, int ldy, const float *x, int ldx, const void *w, int dtype, int M, int N, int K, float alpha,
                                yalm_stream_t s) {
	if (!y || !x || !w || M < 1 || N < 1 || K < 1 || ldy < N || ldx < K) return YALM_EINVAL;
	cudaStream_t st = (cudaStream_t)s;
	if (M <= 2 * kLinMB) {
		const bool vec = row_vec(w, K, dtype) && aligned16(x) && ldx % 4 == 0;
		DISPATCH_DT(dtype, (linear_few_kernel<DT><<<dim3((N + 7) / 8, (M + kLinMB - 1) / kLinMB), 256, 0, st>>>(y, ldy, x, ldx, w, M, N, K, alpha, vec)));
	} else {
		DISPATCH_DT(dtype, (linear_tiled_kernel<DT><<<dim3((N + 63) / 64, (M + 63) / 64), 256, 0, st>>>(y, ldy, x, ldx, w, M, N, K, alpha)));
	}
	return (int)cudaGetLastError();
}

// out16 (M, K) = x (M, ldx) rounded to bf16 (bf16 != 0) or fp16
extern "C" int yalm_cast_rows16(void *out16, const float *x, int ldx, int M, int K, int bf16, yalm_stream_t s) {
	if (!out16 || !x || M < 1 || K < 1) return YALM_EINVAL;
	if (bf16) cast_rows_kernel<__nv_bfloat16><<<M, 256, 0, (cudaStream_t)s>>>(static_cast<__nv_bfloat16 *>(out16), x, ldx, K);
	else cast_rows_kernel<__half><<<M, 256, 0, (cudaStream_t)s>>>(static_cast<__half *>(out16), x, ldx, K);
	return (int)cudaGetLastError();
}

// cache_f32 != 0: fp32 key / value ring, else bf16.
extern "C" int yalm_qkv_post_rows(float *qkv, int ld, void *key_ring, void *value_ring, float *vfirst, int ldvf, const float *qnorm,
                                  const float *knorm, const float *vmix, int vmode, int n, int n_heads, int n_kv, int dk, int dv, int ring,
                                  float eps, int cache_f32, int pos0, const int *ctl, yalm_stream_t s) {
	if (!qkv || !key_ring || !value_ring || n < 1 || ring < 1 || (vmode && !vfirst) || (vmode == 2 && !vmix)) return YALM_EINVAL;
	const int nq = n_heads * dk, nk = n_kv * dk, nv = n_kv * dv;
	cudaStream_t st = (cudaStream_t)s;
	if (cache_f32)
		qkv_post_rows_kernel<float><<<n, 256, 0, st>>>(qkv, ld, (float *)key_ring, (float *)value_ring, vfirst, ldvf, qnorm, knorm, vmix, vmode, nq, nk,
		                                               nv, dk, dv, ring, eps, pos0, ctl);
	else
		qkv_post_rows_kernel<__nv_bfloat16><<<n, 256, 0, st>>>(qkv, ld, (__nv_bfloat16 *)key_ring, (__nv_bfloat16 *)value_ring, vfirst, ldvf, qnorm,
		                                                       knorm, vmix, vmode, nq, nk, nv, dk, dv, ring, eps, pos0, ctl);
	return (int)cudaGetLastError();
}

extern "C" int yalm_kv_pool_rows(float *key_pool, float *value_pool, const void *key_ring, const void *value_ring, int n, int n_kv, int dk, int dv,
                                 int ring, int pool, int max_blocks, int cache_f32, int pos0, const int *ctl, yalm_stream_t s) {
	if (!key_pool || !value_pool || !key_ring || !value_ring || n < 1 || pool < 1 || max_blocks < 1) return YALM_EINVAL;
	const dim3 grid(n / pool + 1, n_kv);
	cudaStream_t st = (cudaStream_t)s;
	if (cache_f32)
		kv_pool_rows_kernel<float><<<grid, 128, 0, st>>>(key_pool, value_pool, (const float *)key_ring, (const float *)value_ring, n, dk, dv, ring, pool,
		                                                 max_blocks, pos0, ctl);
	else
		kv_pool_rows_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(key_pool, value_pool, (const __nv_bfloat16 *)key_ring, (const __nv_bfloat16 *)value_ring,
		                                                         n, dk, dv, ring, pool, max_blocks, pos0, ctl);
	return (int)cudaGetLastError();
}

// Floats of workspace yalm_attn_window_pool wants for value size dv (split partials of decode-sized calls).
extern "C" size_t yalm_attn_window_pool_workspace(int dv) {
	return (size_t)kAttnMaxParts * (dv + 2);
}

static bool lanes_size(int d) { return d >= 8 && d <= 256 && (d & (d - 1)) == 0; }
static bool attn_lanes_off() { // YALM_STACK_ATTN_LANES=0: A/B against the lane-per-key kernel
	static const bool off = [] { const char *e = getenv("YALM_STACK_ATTN_LANES"); return e && e[0] == '0'; }();
	return off;
}
template <int R>
static int launch_attn_lanes(float *out, int ldo, const float *q, int ldq, const void *kr, const void *vr, const float *kp, const float *vp, float *ws,
                             int n, int n_heads, int n_kv, int dk, int dv, int ring, int max_blocks, int window, int pool, float scale, int nsplit,
                             int pos0, const int *ctl, const float *sink, int v_heads, cudaStream_t st) {
	const int rep = n_heads / n_kv, hg = (rep + R - 1) / R;
	const size_t smem = sizeof(float) * ((size_t)R * dk + (size_t)kAttnWarps * R * dv + kAttnWarps * R * 2 + kAttnWarps * R * 32);
	if (smem > 48 * 1024) return YALM_EINVAL;
	attn_window_pool_lanes_kernel<R><<<dim3(n_kv * hg, n, nsplit), kAttnWarps * 32, smem, st>>>(
	    out, ldo, q, ldq, (const __nv_bfloat16 *)kr, (const __nv_bfloat16 *)vr, kp, vp, nsplit > 1 ? ws : nullptr, n_heads, n_kv, dk, dv, ring, max_blocks,
	    window, pool, scale, pos0, ctl, sink, v_heads);
	if (nsplit > 1) attn_merge_kernel<<<dim3(n_heads, n), 128, 0, st>>>(out, ldo, ws, n_heads, dv, nsplit, sink);
	return (int)cudaGetLastError();
}

template <typename CT, int R, int DVC>
static int launch_attn_wp(float *out, int ldo, const float *q, int ldq, const void *kr, const void *vr, const float *kp, const float *vp, float *ws,
                          int n, int n_heads, int n_kv, int dk, int dv, int ring, int max_blocks, int window, int pool, float scale, int nsplit,
                          int pos0, const int *ctl, int ldk, int ldv, const float *sink, int v_heads, cudaStream_t st) {
	const int rep = n_heads / n_kv, hg = (rep + R - 1) / R;
	const size_t smem = sizeof(float) * ((size_t)R * ((dk + 7) & ~7) + (size_t)kAttnWarps * R * dv + kAttnWarps * R * 2);
	if (smem > 160 * 1024) return YALM_EINVAL;
	if (smem > 48 * 1024) YALM_TRY(cudaFuncSetAttribute(attn_window_pool_kernel<CT, R, DVC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
	attn_window_pool_kernel<CT, R, DVC><<<dim3(n_kv * hg, n, nsplit), kAttnWarps * 32, smem, st>>>(
	    out, ldo, q, ldq, (const CT *)kr, (const CT *)vr, kp, vp, nsplit > 1 ? ws : nullptr, n_heads, n_kv, dk, dv, ring, max_blocks, window, pool, scale,
	    pos0, ctl, ldk, ldv, sink, v_heads);
	if (nsplit > 1) attn_merge_kernel<<<dim3(n_heads, n), 128, 0, st>>>(out, ldo, ws, n_heads, dv, nsplit, sink);
	return (int)cudaGetLastError();
}

// workspace: yalm_attn_window_pool_workspace(dv) floats, or null (never split).  context: the most positions a sequence
// reaches (bounds the number of keys when the position lives on the device); 0: unknown.
extern "C" int yalm_attn_window_pool(float *out, int ldo, const float *q, int ldq, const void *key_ring, const void *value_ring, const float *key_pool,
                                     const float *value_pool, float *workspace, int n, int n_heads, int n_kv, int dk, int dv, int ring, int max_blocks,
                                     int window, int pool, float scale, int cache_f32, int context, int pos0, const int *ctl, yalm_stream_t s) {
	return yalm_attn_window_pool_strided(out, ldo, q, ldq, key_ring, dk, value_ring, dv, key_pool, value_pool, workspace, n, n_heads, n_kv, dk, dv, ring,
	                                     max_blocks, window, pool, scale, cache_f32, context, pos0, ctl, s);
}

// The same with explicit row strides of the rings (in elements): values may live inside the key rows (value_ring = key_ring,
// ldv = ldk, the first dv channels of a row), as a cache of shared key / value latents has them.
extern "C" int yalm_attn_window_pool_strided(float *out, int ldo, const float *q, int ldq, const void *key_ring, int ldk, const void *value_ring, int ldv,
                                             const float *key_pool, const float *value_pool, float *workspace, int n, int n_heads, int n_kv, int dk, int dv,
                                             int ring, int max_blocks, int window, int pool, float scale, int cache_f32, int context, int pos0,
                                             const int *ctl, yalm_stream_t s) {
	return yalm_attn_window_pool_sink(out, ldo, q, ldq, key_ring, ldk, value_ring, ldv, key_pool, value_pool, workspace, n, n_heads, n_kv, dk, dv, ring,
	                                  max_blocks, window, pool, scale, cache_f32, context, pos0, ctl, nullptr, n_kv, s);
}

// The same with a sink per query head in the softmax's denominator (sink null: none) and with v_heads value heads for n_kv key
// heads (key head g reads value head g % v_heads: several maps over the same values).
extern "C" int yalm_attn_window_pool_sink(float *out, int ldo, const float *q, int ldq, const void *key_ring, int ldk, const void *value_ring, int ldv,
                                          const float *key_pool, const float *value_pool, float *workspace, int n, int n_heads, int n_kv, int dk, int dv,
                                          int ring, int max_blocks, int window, int pool, float scale, int cache_f32, int context, int pos0, const int *ctl,
                                          const float *sink, int v_heads, yalm_stream_t s) {
	if (!out || !q || !key_ring || !value_ring || n < 1 || n_kv < 1 || n_heads % n_kv || dv > 512 || ldk < dk || ldv < dv ||
	    (pool > 0 && (!key_pool || !value_pool)) || v_heads < 1 || n_kv % v_heads)
		return YALM_EINVAL;
	cudaStream_t st = (cudaStream_t)s;
	const int rep = n_heads / n_kv, R = rep >= 2 ? 4 : 1, hg = (rep + R - 1) / R;
	// few CTAs (decoding): split the keys so that every SM has work; the count depends on shapes only, never on the position
	int nsplit = 1;
	const int ctas = n_kv * hg * n;
	if (workspace && ctas < 296) {
		const int most_keys = window > 0 ? window + (pool > 0 ? max_blocks : 0) : (context > 0 ? context : ring);
		const int tiles = (most_keys + 31) / 32 + 1;
		nsplit = std::min({(296 + ctas - 1) / ctas, std::max(1, (tiles + kAttnWarps - 1) / kAttnWarps), std::max(1, kAttnMaxParts / (n * n_heads)), 64});
	}
	if (!cache_f32 && ldk == dk && ldv == dv && lanes_size(dk) && lanes_size(dv) && aligned16(key_ring) && aligned16(value_ring) && aligned16(key_pool) && aligned16(value_pool) &&
	    !attn_lanes_off()) {
		// heads per CTA: four share every key read; with few CTAs (decoding) a warp's instruction chain, not the reads, sets the
		// time, so fewer heads per CTA spread the same work over more SMs (the keys then come from the L2 more than once)
		int RL = R;
		while (RL > 1 && (long)n_kv * ((rep + RL - 1) / RL) * n * nsplit < device_info().sms) RL >>= 1;
#define LANES_CASE(R_)                                                                                                                \
	return launch_attn_lanes<R_>(out, ldo, q, ldq, key_ring, value_ring, key_pool, value_pool, workspace, n, n_heads, n_kv, dk, dv, ring, max_blocks, window, \
	                             pool, scale, nsplit, pos0, ctl, sink, v_heads, st)
		if (RL == 1) LANES_CASE(1);
		if (RL == 2) LANES_CASE(2);
		LANES_CASE(4);
#undef LANES_CASE
	}
#define ATTN_CASE(CT, R_, DVC_)                                                                                                       \
	return launch_attn_wp<CT, R_, DVC_>(out, ldo, q, ldq, key_ring, value_ring, key_pool, value_pool, workspace, n, n_heads, n_kv, dk, dv, ring, max_blocks, \
	                                    window, pool, scale, nsplit, pos0, ctl, ldk, ldv, sink, v_heads, st)
#define ATTN_DVC(CT, R_)                                                                                                              \
	if (dv <= 64) ATTN_CASE(CT, R_, 2);                                                                                               \
	else if (dv <= 128) ATTN_CASE(CT, R_, 4);                                                                                         \
	else if (dv <= 256) ATTN_CASE(CT, R_, 8);                                                                                         \
	else ATTN_CASE(CT, R_, 16)
	if (cache_f32) {
		if (R == 1) { ATTN_DVC(float, 1); }
		else { ATTN_DVC(float, 4); }
	} else {
		if (R == 1) { ATTN_DVC(__nv_bfloat16, 1); }
		else { ATTN_DVC(__nv_bfloat16, 4); }
	}
#undef ATTN_DVC
#undef ATTN_CASE
}

extern "C" int yalm_norm_residual_rows(float *x, const float *y, int ldy, int nsum, const float *w, float w_offset, float eps, int n, int dim,
                                       yalm_stream_t s) {
	if (!x || !y || !w || n < 1 || nsum < 1 || dim < 1 || (size_t)dim * 4 > 48 * 1024) return YALM_EINVAL;
	norm_residual_rows_kernel<<<n, 256, sizeof(float) * dim, (cudaStream_t)s>>>(x, y, ldy, nsum, w, w_offset, eps, dim);
	return (int)cudaGetLastError();
}

extern "C" int yalm_norm_gather_rows(float *out, const float *x, const int *rows, const float *w, int scalar_weight, float w_offset, float eps, int n_rows,
                                     int dim, yalm_stream_t s) {
	if (!out || !x || !w || n_rows < 1) return YALM_EINVAL;
	norm_gather_rows_kernel<<<n_rows, 256, 0, (cudaStream_t)s>>>(out, x, rows, w, scalar_weight, w_offset, eps, dim);
	return (int)cudaGetLastError();
}

// act: YALM_ACT_GELU, YALM_ACT_SILU, or 2 = g * sigmoid(alpha g)
extern "C" int yalm_glu_act_rows(float *h, const float *gu, int n, int ff, int act, float alpha, float limit, float up_offset, yalm_stream_t s) {
	if (!h || !gu || n < 1 || ff < 1) return YALM_EINVAL;
	glu_act_rows_kernel<<<dim3((ff + 255) / 256, n), 256, 0, (cudaStream_t)s>>>(h, gu, ff, act, alpha, limit, up_offset);
	return (int)cudaGetLastError();
}

// score: 0 softmax, 1 sigmoid
extern "C" int yalm_router_topk_rows(int *ids, float *wts, const float *x, int ldx, const void *wr, int dtype, int n, int n_experts, int top, int dim,
                                     int score, int renorm, float renorm_eps, int groups, int keep_groups, yalm_stream_t s) {
	return yalm_router_bias_topk_rows(ids, wts, x, ldx, wr, dtype, n, n_experts, top, dim, score, renorm, renorm_eps, groups, keep_groups, nullptr, 1.f, s);
}

// bias (n_experts, optional): the experts are chosen by score + bias, the weights use the score alone; weight_scale multiplies
// the (renormalised) weights.
extern "C" int yalm_router_bias_topk_rows(int *ids, float *wts, const float *x, int ldx, const void *wr, int dtype, int n, int n_experts, int top, int dim,
                                          int score, int renorm, float renorm_eps, int groups, int keep_groups, const float *bias, float weight_scale,
                                          yalm_stream_t s) {
	if (!ids || !wts || !x || !wr || n < 1 || top < 1 || top > n_experts || n_experts > 1024 || groups < 1 || n_experts % groups || keep_groups < 1 ||
	    keep_groups > groups || top > keep_groups * (n_experts / groups))
		return YALM_EINVAL;
	const bool vec = row_vec(wr, dim, dtype) && aligned16(x) && ldx % 4 == 0;
	DISPATCH_DT(dtype, (router_topk_rows_kernel<DT><<<n, n <= 4 ? 256 : 128, sizeof(float) * (2 * n_experts + groups), (cudaStream_t)s>>>(
	                       ids, wts, x, ldx, wr, n_experts, top, dim, score, renorm, renorm_eps, groups, keep_groups, vec, bias, weight_scale)));
	return (int)cudaGetLastError();
}

extern "C" int yalm_moe_glu_slots(float *h, const float *x, int ldx, const void *wg, const void *wu, int dtype, const int *ids, const float *wts, int n,
                                  int top, int ff, int dim, int act, float alpha, float limit, float up_offset, int in_scale, yalm_stream_t s) {
	return yalm_moe_glu_slots_real(h, x, ldx, wg, wu, dtype, ids, wts, n, top, ff, dim, act, alpha, limit, up_offset, in_scale, 1 << 30, s);
}
extern "C" int yalm_moe_down_slots(float *y, int ldy, const float *h, const void *wd, int dtype, const int *ids, const float *wts, int n, int top, int ff,
                                   int dim, int out_scale, yalm_stream_t s) {
	return yalm_moe_down_slots_real(y, ldy, h, wd, dtype, ids, wts, n, top, ff, dim, out_scale, 1 << 30, nullptr, 0, s);
}

// The same with identity experts: ids >= n_real have no matrices, their slot's output is the row of x itself (times the weight).
extern "C" int yalm_moe_glu_slots_real(float *h, const float *x, int ldx, const void *wg, const void *wu, int dtype, const int *ids, const float *wts, int n,
                                       int top, int ff, int dim, int act, float alpha, float limit, float up_offset, int in_scale, int n_real,
                                       yalm_stream_t s) {
	if (!h || !x || !wg || !wu || !ids || !wts || n < 1 || top < 1) return YALM_EINVAL;
	const bool vec = row_vec(wg, dim, dtype) && row_vec(wu, dim, dtype) && aligned16(x) && ldx % 4 == 0;
	DISPATCH_DT(dtype, (moe_glu_slots_kernel<DT><<<dim3((ff + 3) / 4, n * top), 128, 0, (cudaStream_t)s>>>(h, x, ldx, wg, wu, ids, wts, top, ff, dim, act,
	                                                                                                     alpha, limit, up_offset, in_scale, vec, n_real)));
	return (int)cudaGetLastError();
}

extern "C" int yalm_moe_down_slots_real(float *y, int ldy, const float *h, const void *wd, int dtype, const int *ids, const float *wts, int n, int top,
                                        int ff, int dim, int out_scale, int n_real, const float *x, int ldx, yalm_stream_t s) {
	if (!y || !h || !wd || !ids || !wts || n < 1 || top < 1 || (n_real < (1 << 30) && !x)) return YALM_EINVAL;
	const bool vec = row_vec(wd, ff, dtype) && aligned16(h) && ff % 4 == 0;
	DISPATCH_DT(dtype, (moe_down_slots_kernel<DT><<<dim3((dim + 3) / 4, n * top), 128, 0, (cudaStream_t)s>>>(y, ldy, h, wd, ids, wts, ff, dim, out_scale, vec, n_real, x, ldx, top)));
	return (int)cudaGetLastError();
}

extern "C" int yalm_moe_identity_slots(float *y, int ldy, const float *x, int ldx, const int *ids, const float *wts, int n, int top, int dim, int n_real,
                                       int out_scale, yalm_stream_t s) {
	if (!y || !x || !ids || !wts || n < 1 || top < 1 || dim < 1) return YALM_EINVAL;
	moe_identity_slots_kernel<<<n * top, 256, 0, (cudaStream_t)s>>>(y, ldy, x, ldx, ids, wts, top, dim, n_real, out_scale);
	return (int)cudaGetLastError();
}

// Slots sorted by expert (order[j] = slot at place j): the A operand of the per-expert tensor-core products, and the way back.
extern "C" int yalm_moe_gather_rows16(void *out16, const float *x, int ldx, const int *order, const float *wts, int n_slots, int top, int dim,
                                      int bf16, int in_scale, yalm_stream_t s) {
	if (!out16 || !x || !order || !wts || n_slots < 1 || top < 1 || dim < 1) return YALM_EINVAL;
	if (bf16) moe_gather_rows_kernel<__nv_bfloat16><<<n_slots, 256, 0, (cudaStream_t)s>>>(static_cast<__nv_bfloat16 *>(out16), x, ldx, order, wts, top, dim, in_scale);
	else moe_gather_rows_kernel<__half><<<n_slots, 256, 0, (cudaStream_t)s>>>(static_cast<__half *>(out16), x, ldx, order, wts, top, dim, in_scale);
	return (int)cudaGetLastError();
}
extern "C" int yalm_moe_scatter_rows(float *y, int ldy, const float *ys, int lds, const int *order, const float *wts, int n_slots, int dim,
                                     int out_scale, yalm_stream_t s) {
	if (!y || !ys || !order || !wts || n_slots < 1 || dim < 1) return YALM_EINVAL;
	moe_scatter_rows_kernel<<<n_slots, 256, 0, (cudaStream_t)s>>>(y, ldy, ys, lds, order, wts, dim, out_scale);
	return (int)cudaGetLastError();
}
