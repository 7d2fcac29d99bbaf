// Row-batched ops of the layered executor (stack.cpp) for layers that carry per-sequence state besides a key / value ring:
// token shift, short causal convolutions, linear recurrences over a matrix state (state-space and gated-delta-rule mixers),
// and the sigmoid-weighted windowed attention.  As in ops_stack.cu every op takes M rows = M consecutive positions of one
// sequence (M = 1: a decode step; M > 1: a portion of a prompt cut anywhere) and runs the same arithmetic for both; what a
// sequence carries from one call to the next lives in fp32 state buffers owned by the model.  A call whose first position
// is 0 starts a sequence: the stored state is ignored (taken as zero), so giving a sequence's state back needs no clearing.
//
// Mechanisms (constants are parameters):
//   norm_shift_rows        h = rms(x) * w (one weight per channel or one number) and, optionally, the token-shifted copy
//                          hs = h + (h of the previous position - h) * mu
//   conv_act_rows          per-channel causal convolution over the last `taps` positions (+ bias) and SiLU
//   state_scan_rows        M <- a * M;  e = beta (v - M^T k)  or  e = vscale * v;  M <- M + k e^T;  y = M^T q (+ skip * v)
//                          with a scalar or per-key-channel decay: both the state-space recurrence and the gated delta rule
//   ssm_prep_rows          dt = softplus(raw + bias), decay = exp(-exp(A_log) dt)
//   delta_prep_rows        unit q / k per head, beta = sigmoid(raw), per-channel decay from raw step sizes
//   gated_group_norm_rows  rms over equal parts of (y * silu(z)), times a weight
//   head_norm_gate_rows    per head rms(o) * w * sigmoid(gate)
//   qk_bias_append_rows    projection biases, key append to the ring and to the kept-first buffer
//   attn_sigmoid_rows      window + kept first tokens, weights sigmoid(q.k scale + distance bias + head bias), values = keys,
//                          sigmoid output gate
//   residual_sum_rows      x += a (+ b) + sum of partial outputs
//   softcap_rows           z <- cap * tanh(z / cap)
#include "common.cuh"

#include <cuda_bf16.h>

#include <algorithm>
#include <cstdlib>

#include "launch.h"
#include "stack_rows.cuh"

namespace yalm {
namespace stack {

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float siluf_(float z) { return z / (1.0f + expf(-z)); }

// ---- norm + token shift --------------------------------------------------------------------------------------------------
// One CTA per row.  The previous position's h of row m > 0 is recomputed from x[m - 1]; row 0 takes it from `state` (zero at
// position 0).  update != 0 (single-row calls only: no other CTA reads the state): the row's h becomes the state; calls with
// more rows copy their last h row afterwards.  h may alias x only when hs is null.
__global__ void __launch_bounds__(256) norm_shift_rows_kernel(float *__restrict__ h, float *__restrict__ hs, const float *x, const float *__restrict__ w,
                                                              int scalar, float woff, float eps, const float *__restrict__ mu, float *state, int update,
                                                              int dim, int pos0, const int *__restrict__ ctl) {
	__shared__ float red[33];
	const int m = blockIdx.x, p = first_pos(ctl, pos0) + m;
	const float *xr = x + (size_t)m * dim, *xp = xr - dim;
	float ss = 0.f, sp = 0.f;
	for (int e = threadIdx.x; e < dim; e += blockDim.x) {
		ss += xr[e] * xr[e];
		if (hs && m > 0) sp += xp[e] * xp[e];
	}
	ss = block_sum(ss, red);
	const float r = 1.0f / sqrtf(ss / dim + eps);
	float rp = 0.f;
	if (hs && m > 0) rp = 1.0f / sqrtf(block_sum(sp, red) / dim + eps);
	for (int e = threadIdx.x; e < dim; e += blockDim.x) {
		const float g = woff + (scalar ? w[0] : w[e]);
		const float v = xr[e] * r * g;
		if (hs) {
			const float prev = m > 0 ? xp[e] * rp * g : (p > 0 ? state[e] : 0.f);
			hs[(size_t)m * dim + e] = v + (prev - v) * mu[e];
			if (update) state[e] = v;
		}
		h[(size_t)m * dim + e] = v;
	}
}

// ---- short causal convolution + SiLU ---------------------------------------------------------------------------------------
// out[m, c] = silu(b[c] + sum_j w[c, j] in[m - (taps - 1) + j, c]); rows before the call's first come from the state
// (C, taps - 1), which holds the inputs of positions p0 - (taps - 1) .. p0 - 1; positions before 0 are zero.
__device__ __forceinline__ float conv_input(const float *in, int ldi, const float *state, int c, int taps, int row, int p0) {
	if (row >= 0) return in[(size_t)row * ldi + c];
	return p0 + row >= 0 ? state[(size_t)c * (taps - 1) + (taps - 1) + row] : 0.f;
}
// new state slot s = the input of row n - (taps - 1) + s; ascending s only reads old slots above s
__device__ __forceinline__ void conv_state_update(const float *in, int ldi, float *state, int c, int taps, int n, int p0) {
	for (int s = 0; s < taps - 1; ++s) state[(size_t)c * (taps - 1) + s] = conv_input(in, ldi, state, c, taps, n - (taps - 1) + s, p0);
}
constexpr int kConvRows = 32;
__global__ void __launch_bounds__(128) conv_act_rows_kernel(float *__restrict__ out, int ldo, const float *__restrict__ in, int ldi,
                                                            const float *__restrict__ w, const float *__restrict__ bias, float *state, int n, int C,
                                                            int taps, int pos0, const int *__restrict__ ctl) {
	const int c = blockIdx.x * blockDim.x + threadIdx.x;
	if (c >= C) return;
	const int p0 = first_pos(ctl, pos0);
	const int m0 = blockIdx.y * kConvRows, m1 = min(n, m0 + kConvRows);
	const float b = bias ? bias[c] : 0.f;
	for (int m = m0; m < m1; ++m) {
		float acc = b;
		for (int j = 0; j < taps; ++j) acc = fmaf(w[(size_t)c * taps + j], conv_input(in, ldi, state, c, taps, m - (taps - 1) + j, p0), acc);
		out[(size_t)m * ldo + c] = siluf_(acc);
	}
	if (gridDim.y == 1) conv_state_update(in, ldi, state, c, taps, n, p0); // this thread is the only reader of its channel's state
}
__global__ void __launch_bounds__(128) conv_state_rows_kernel(const float *__restrict__ in, int ldi, float *state, int n, int C, int taps, int pos0,
                                                              const int *__restrict__ ctl) {
	const int c = blockIdx.x * blockDim.x + threadIdx.x;
	if (c < C) conv_state_update(in, ldi, state, c, taps, n, first_pos(ctl, pos0));
}

// ---- linear recurrence over a matrix state -----------------------------------------------------------------------------------
// Per head a (D, P) matrix M whose columns evolve independently:
//   M <- a * M       (the decay a: one number per head, or one per head and key channel, acting on rows)
//   e = beta * (v - M^T k)   (delta rule)   or   e = vscale * v
//   M <- M + k e^T;   y = M^T q  (+ skip * v)
// One CTA owns 16 columns of one head; 8 neighbouring lanes share a column, lane `sub` holding the EPL consecutive rows
// sub * EPL .. in registers, so the two dot products of a step are EPL multiply-adds (four partial sums) and three shuffles.
// k, q, the decays and v of 8 positions at a time go global -> shared with cp.async into one of two stages: the next 8 load
// while these are consumed.  In shared memory a position's row is cut into the 8 lanes' segments, padded so that the lanes'
// 16-byte reads fall into different banks.  The reduction of a position's output is carried into the next position's step,
// where it shares the shuffle rounds of that step's M^T k, so only the recurrence itself (decay, M^T k, update) is a serial
// chain.  The order of every sum is fixed, so a position's output does not depend on how the rows were cut into calls.
// State in global memory: (head, column, row) fp32.
struct ScanArgs {
	float *out;
	int ldo;
	const float *k, *q, *v, *decay, *vscale, *beta, *skip;
	int ldk, ldq, ldv, ldd, ldvs, ldb;
	int decay_per_channel;
	float *state;
	int n, H, rep, D, P, pos0;
	const int *ctl;
	int vec; // k, q and per-channel decay rows are 16-byte aligned: 16-byte copies
};
constexpr int kScanCols = 16, kScanTok = 8, kScanMaxD = 256;

__device__ __forceinline__ void cp_async4(float *smem, const float *gmem) {
	asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async16f(float *smem, const float *gmem) {
	asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}

template <int EPL>
struct ScanLayout {
	static constexpr int SEG = EPL + (EPL >= 8 ? 4 : 0); // floats between two lanes' segments of a row
	static constexpr int DP = 8 * SEG;
	static constexpr int STAGE = 3 * kScanTok * DP + kScanTok * kScanCols + kScanTok * 4; // k, q, decay rows; v; (decay, vscale, beta) per position
};

// EPL consecutive floats of a shared-memory segment into registers, with the widest aligned reads
template <int EPL>
__device__ __forceinline__ void load_seg(float (&r)[EPL], const float *p) {
	if constexpr (EPL % 4 == 0) {
#pragma unroll
		for (int e = 0; e < EPL; e += 4) {
			const float4 v = *reinterpret_cast<const float4 *>(p + e);
			r[e] = v.x, r[e + 1] = v.y, r[e + 2] = v.z, r[e + 3] = v.w;
		}
	} else if constexpr (EPL == 2) {
		const float2 v = *reinterpret_cast<const float2 *>(p);
		r[0] = v.x, r[1] = v.y;
	} else
		r[0] = p[0];
}

template <int EPL>
__global__ void __launch_bounds__(kScanCols * 8) state_scan_kernel(ScanArgs a) {
	using LO = ScanLayout<EPL>;
	constexpr int SEG = LO::SEG, DP = LO::DP, TOK = kScanTok, STAGE = LO::STAGE;
	extern __shared__ __align__(16) float scan_sm[];
	const int h = blockIdx.y, kh = h / a.rep, c0 = blockIdx.x * kScanCols;
	const int tid = threadIdx.x, col = tid >> 3, sub = tid & 7;
	const bool live = c0 + col < a.P;
	const bool fresh = first_pos(a.ctl, a.pos0) == 0;
	float *sp = a.state + ((size_t)h * a.P + min(c0 + col, a.P - 1)) * a.D + sub * EPL;
	float s[EPL];
#pragma unroll
	for (int e = 0; e < EPL; ++e) s[e] = (!fresh && sub * EPL + e < a.D) ? sp[e] : 0.f;
	const float skip = a.skip ? a.skip[h] : 0.f;
	// what the copies never write: rows past D, the padding, columns past P, and the defaults of absent per-position scalars
	for (int idx = tid; idx < 2 * STAGE; idx += blockDim.x) {
		const int r = idx % STAGE;
		scan_sm[idx] = (r >= 3 * TOK * DP + TOK * kScanCols && (r - 3 * TOK * DP - TOK * kScanCols) % 4 < 2) ? 1.f : 0.f;
	}
	__syncthreads();
	auto issue = [&](int t0, int stage) {
		float *ks = scan_sm + stage * STAGE, *qs = ks + TOK * DP, *gs = qs + TOK * DP, *vs = gs + TOK * DP, *sc = vs + TOK * kScanCols;
		const int tc = min(TOK, a.n - t0);
		if (a.vec && EPL >= 4) {
			const int D4 = a.D >> 2;
			for (int idx = tid; idx < tc * D4; idx += blockDim.x) {
				const int t = idx / D4, i = (idx % D4) * 4, at = t * DP + (i / EPL) * SEG + i % EPL;
				cp_async16f(ks + at, a.k + (size_t)(t0 + t) * a.ldk + kh * a.D + i);
				cp_async16f(qs + at, a.q + (size_t)(t0 + t) * a.ldq + kh * a.D + i);
				if (a.decay_per_channel) cp_async16f(gs + at, a.decay + (size_t)(t0 + t) * a.ldd + h * a.D + i);
			}
		} else {
			for (int idx = tid; idx < tc * a.D; idx += blockDim.x) {
				const int t = idx / a.D, i = idx % a.D, at = t * DP + (i / EPL) * SEG + i % EPL;
				cp_async4(ks + at, a.k + (size_t)(t0 + t) * a.ldk + kh * a.D + i);
				cp_async4(qs + at, a.q + (size_t)(t0 + t) * a.ldq + kh * a.D + i);
				if (a.decay_per_channel) cp_async4(gs + at, a.decay + (size_t)(t0 + t) * a.ldd + h * a.D + i);
			}
		}
		for (int idx = tid; idx < tc * kScanCols; idx += blockDim.x) {
			const int t = idx / kScanCols, c = idx % kScanCols;
			if (c0 + c < a.P) cp_async4(vs + idx, a.v + (size_t)(t0 + t) * a.ldv + h * a.P + c0 + c);
		}
		if (tid < tc) {
			if (!a.decay_per_channel) cp_async4(sc + tid * 4, a.decay + (size_t)(t0 + tid) * a.ldd + h);
			if (a.vscale) cp_async4(sc + tid * 4 + 1, a.vscale + (size_t)(t0 + tid) * a.ldvs + h);
			if (a.beta) cp_async4(sc + tid * 4 + 2, a.beta + (size_t)(t0 + tid) * a.ldb + h);
		}
		asm volatile("cp.async.commit_group;" ::: "memory");
	};
	float po = 0.f, pvv = 0.f; // the previous position's output: partial sum of this lane, and its v
	float *pout = nullptr;
	issue(0, 0);
	for (int c = 0, t0 = 0; t0 < a.n; ++c, t0 += TOK) {
		const int tc = min(TOK, a.n - t0);
		if (t0 + TOK < a.n) {
			issue(t0 + TOK, (c + 1) & 1);
			asm volatile("cp.async.wait_group 1;" ::: "memory");
		} else
			asm volatile("cp.async.wait_group 0;" ::: "memory");
		__syncthreads();
		const float *ks = scan_sm + (c & 1) * STAGE, *qs = ks + TOK * DP, *gs = qs + TOK * DP, *vs = gs + TOK * DP, *sc = vs + TOK * kScanCols;
		for (int t = 0; t < tc; ++t) {
			float kt[EPL], qt[EPL];
			load_seg<EPL>(kt, ks + t * DP + sub * SEG);
			load_seg<EPL>(qt, qs + t * DP + sub * SEG);
			const float vv = vs[t * kScanCols + col];
			if (a.decay_per_channel) {
				float gt[EPL];
				load_seg<EPL>(gt, gs + t * DP + sub * SEG);
#pragma unroll
				for (int e = 0; e < EPL; ++e) s[e] *= gt[e];
			} else {
				const float d = sc[t * 4];
#pragma unroll
				for (int e = 0; e < EPL; ++e) s[e] *= d;
			}
			float u;
			if (a.beta) {
				float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
				for (int e = 0; e < EPL; ++e) d4[e & 3] = fmaf(s[e], kt[e], d4[e & 3]);
				float dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
				dot += __shfl_xor_sync(kFull, dot, 4), po += __shfl_xor_sync(kFull, po, 4);
				dot += __shfl_xor_sync(kFull, dot, 2), po += __shfl_xor_sync(kFull, po, 2);
				dot += __shfl_xor_sync(kFull, dot, 1), po += __shfl_xor_sync(kFull, po, 1);
				u = sc[t * 4 + 2] * (vv - dot);
			} else {
				po += __shfl_xor_sync(kFull, po, 4), po += __shfl_xor_sync(kFull, po, 2), po += __shfl_xor_sync(kFull, po, 1);
				u = sc[t * 4 + 1] * vv;
			}
			if (pout && sub == 0 && live) *pout = po + skip * pvv;
			float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
			for (int e = 0; e < EPL; ++e) {
				s[e] = fmaf(kt[e], u, s[e]);
				o4[e & 3] = fmaf(s[e], qt[e], o4[e & 3]);
			}
			po = (o4[0] + o4[1]) + (o4[2] + o4[3]), pvv = vv;
			pout = a.out + (size_t)(t0 + t) * a.ldo + h * a.P + min(c0 + col, a.P - 1);
		}
		__syncthreads(); // this stage is consumed: the copies of the position group after next may land in it
	}
	po += __shfl_xor_sync(kFull, po, 4), po += __shfl_xor_sync(kFull, po, 2), po += __shfl_xor_sync(kFull, po, 1);
	if (pout && sub == 0 && live) *pout = po + skip * pvv;
	if (live) {
#pragma unroll
		for (int e = 0; e < EPL; ++e)
			if (sub * EPL + e < a.D) sp[e] = s[e];
	}
}

// dt[m, h] = softplus(dt + bias[h]) in place; decay[m, h] = exp(-exp(a_log[h]) * dt)
__global__ void ssm_prep_rows_kernel(float *__restrict__ dt, int lddt, float *__restrict__ decay, int ldd, const float *__restrict__ bias,
                                     const float *__restrict__ a_log, int H) {
	const int m = blockIdx.x;
	for (int h = threadIdx.x; h < H; h += blockDim.x) {
		const float d = softplusf_(dt[(size_t)m * lddt + h] + bias[h]);
		dt[(size_t)m * lddt + h] = d;
		decay[(size_t)m * ldd + h] = expf(-expf(a_log[h]) * d);
	}
}

// One CTA per row.  q, k (G heads of D, row stride ldqk, in place): x / sqrt(sum x^2 + unit_eps), q also times q_scale.
// beta (H, in place) = sigmoid(raw).  g (H * D, in place) = exp(-exp(a_log[h]) * softplus(raw + dt_bias)).
__global__ void __launch_bounds__(256) delta_prep_rows_kernel(float *__restrict__ q, float *__restrict__ k, int ldqk, float *__restrict__ beta, int ldb,
                                                              float *__restrict__ g, int ldg, const float *__restrict__ a_log,
                                                              const float *__restrict__ dt_bias, int H, int G, int D, float unit_eps, float q_scale) {
	const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
	for (int j = warp; j < 2 * G; j += nw) {
		float *row = (j < G ? q + (size_t)m * ldqk + j * D : k + (size_t)m * ldqk + (j - G) * D);
		float ss = 0.f;
		for (int i = lane; i < D; i += 32) ss += row[i] * row[i];
		ss = warp_sum(ss);
		const float r = (j < G ? q_scale : 1.f) / sqrtf(ss + unit_eps);
		for (int i = lane; i < D; i += 32) row[i] *= r;
	}
	for (int h = threadIdx.x; h < H; h += blockDim.x) beta[(size_t)m * ldb + h] = sigmoidf_(beta[(size_t)m * ldb + h]);
	for (int e = threadIdx.x; e < H * D; e += blockDim.x) {
		const float step = softplusf_(g[(size_t)m * ldg + e] + dt_bias[e]);
		g[(size_t)m * ldg + e] = expf(-expf(a_log[e / D]) * step);
	}
}

// out[m, c] = rms_part(y[m, c] * silu(z[m, c])) * w[c], the row cut into gridDim.y equal parts.  grid (rows, parts).
__global__ void __launch_bounds__(1024) gated_group_norm_rows_kernel(float *__restrict__ out, int ldo, const float *__restrict__ y, int ldy,
                                                                    const float *__restrict__ z, int ldz, const float *__restrict__ w, int part, float eps) {
	__shared__ float red[33];
	const int m = blockIdx.x, c0 = blockIdx.y * part;
	float ss = 0.f;
	for (int c = threadIdx.x; c < part; c += blockDim.x) {
		const float v = y[(size_t)m * ldy + c0 + c] * siluf_(z[(size_t)m * ldz + c0 + c]);
		ss += v * v;
	}
	ss = block_sum(ss, red);
	const float r = 1.0f / sqrtf(ss / part + eps);
	for (int c = threadIdx.x; c < part; c += blockDim.x)
		out[(size_t)m * ldo + c0 + c] = y[(size_t)m * ldy + c0 + c] * siluf_(z[(size_t)m * ldz + c0 + c]) * r * w[c0 + c];
}

// out[m, h, c] = o / sqrt(mean_c o^2 + eps) * w[c] * sigmoid(gate[m, h, c]); one warp per (row, head), w shared by the heads
__global__ void __launch_bounds__(128) head_norm_gate_rows_kernel(float *__restrict__ out, int ldo, const float *__restrict__ o, int ldi,
                                                                  const float *__restrict__ gate, int ldg, const float *__restrict__ w, int H, int P,
                                                                  float eps, int gate_silu) {
	const int m = blockIdx.y, h = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
	if (h >= H) return;
	const float *row = o + (size_t)m * ldi + h * P;
	float ss = 0.f;
	for (int c = lane; c < P; c += 32) ss += row[c] * row[c];
	ss = warp_sum(ss);
	const float r = 1.0f / sqrtf(ss / P + eps);
	for (int c = lane; c < P; c += 32) {
		const float g = gate[(size_t)m * ldg + h * P + c];
		out[(size_t)m * ldo + h * P + c] = row[c] * r * w[c] * (gate_silu ? siluf_(g) : sigmoidf_(g));
	}
}

// ---- sigmoid attention -----------------------------------------------------------------------------------------------------
// q += qb, k += kb (in place, fp32); k goes to ring slot p % ring and, for the sequence's first `keep` positions, also to the
// kept-first buffer (kv head, keep, channel), which the ring's reuse never touches.
template <typename CT>
__global__ void __launch_bounds__(256) qk_bias_append_rows_kernel(float *__restrict__ q, float *__restrict__ k, int ld, const float *__restrict__ qb,
                                                                  const float *__restrict__ kb, CT *__restrict__ ring_buf, CT *__restrict__ first_buf,
                                                                  int nq, int nk, int dk, int ring, int keep, int pos0, const int *__restrict__ ctl) {
	const int m = blockIdx.x, p = first_pos(ctl, pos0) + m, slot = p % ring;
	if (qb)
		for (int e = threadIdx.x; e < nq; e += blockDim.x) q[(size_t)m * ld + e] += qb[e];
	for (int e = threadIdx.x; e < nk; e += blockDim.x) {
		const float v = k[(size_t)m * ld + e] + (kb ? kb[e] : 0.f);
		k[(size_t)m * ld + e] = v;
		const int g = e / dk, d = e % dk;
		cache_put(ring_buf, ((size_t)g * ring + slot) * dk + d, v);
		if (p < keep) cache_put(first_buf, ((size_t)g * keep + p) * dk + d, v);
	}
}

// Query row m at position i sees the positions lo .. i (lo = max(0, i - window + 1); window 0: lo = 0) from the ring and the
// positions 0 .. min(keep, lo) - 1 from the kept-first buffer, each at its true distance i - j.  The weight of a key is
// sigmoid(q . k * scale + rel[bucket[i - j], h] + hb[h]); weights are not normalised, the values are the keys, and the
// result is multiplied by sigmoid(gate) (gate null: not).  One CTA per (kv head x up to R query heads that share it, row,
// split); its warps take 32-key tiles in turn, lane = key for the scores and lane = channel for the weighted sum.  With
// splits (few rows: decoding) a CTA leaves its partial sum in `part` and attn_sigmoid_merge_kernel adds the splits in order.
constexpr int kSigWarps = 4;
template <typename CT, int R, int DVC>
__global__ void __launch_bounds__(kSigWarps * 32) attn_sigmoid_rows_kernel(float *__restrict__ out, int ldo, const float *__restrict__ q, int ldq,
                                                                           const CT *__restrict__ ring_buf, const CT *__restrict__ first_buf,
                                                                           const float *__restrict__ gate, int ldg, const float *__restrict__ rel,
                                                                           const int *__restrict__ bucket, const float *__restrict__ hb,
                                                                           float *__restrict__ part, int n_heads, int n_kv, int dk, int ring, int window,
                                                                           int keep, float scale, int pos0, const int *__restrict__ ctl) {
	extern __shared__ __align__(16) float sm[];
	const int dkp = (dk + 3) & ~3;
	float *qs = sm;                 // R x dkp
	float *macc = qs + R * dkp;     // kSigWarps x R x dk
	const int rep = n_heads / n_kv, hg = (rep + R - 1) / R;
	const int g = blockIdx.x / hg, h0 = g * rep + (blockIdx.x % hg) * R, nh = min(R, g * rep + rep - h0);
	const int m = blockIdx.y, z = blockIdx.z, nsplit = gridDim.z;
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int i = first_pos(ctl, pos0) + m;
	const int lo = window > 0 ? max(0, i - window + 1) : 0;
	const int nfirst = min(keep, lo), ntok = i - lo + 1;
	for (int e = threadIdx.x; e < R * dkp; e += blockDim.x) {
		const int r = e / dkp, d = e % dkp;
		qs[e] = (r < nh && d < dk) ? q[(size_t)m * ldq + (size_t)(h0 + r) * dk + d] * scale : 0.f;
	}
	__syncthreads();
	const CT *rbase = ring_buf + (size_t)g * ring * dk, *fbase = first_buf ? first_buf + (size_t)g * keep * dk : nullptr;
	float bias_h[R];
#pragma unroll
	for (int r = 0; r < R; ++r) bias_h[r] = (hb && r < nh) ? hb[h0 + r] : 0.f;
	float acc[R][DVC];
#pragma unroll
	for (int r = 0; r < R; ++r)
#pragma unroll
		for (int c = 0; c < DVC; ++c) acc[r][c] = 0.f;
	// kept-first keys and window keys occupy separate 32-key tiles
	const int ftiles = (nfirst + 31) / 32, ntiles = ftiles + (ntok + 31) / 32, per = (ntiles + nsplit - 1) / nsplit;
	const int t_end = min(ntiles, (z + 1) * per);
	for (int t = z * per + warp; t < t_end; t += kSigWarps) {
		const bool first = t < ftiles;
		const int idx0 = first ? t * 32 : (t - ftiles) * 32, cnt = min(32, (first ? nfirst : ntok) - idx0);
		const int j = first ? idx0 + lane : lo + idx0 + lane; // this lane's key position
		float p[R];
#pragma unroll
		for (int r = 0; r < R; ++r) p[r] = 0.f;
		if (lane < cnt) {
			const CT *krow = first ? fbase + (size_t)j * dk : rbase + (size_t)(j % ring) * dk;
			float s[R];
#pragma unroll
			for (int r = 0; r < R; ++r) s[r] = 0.f;
			for (int d = 0; d < dk; ++d) {
				const float kv = cache_get(krow, d);
#pragma unroll
				for (int r = 0; r < R; ++r) s[r] = fmaf(kv, qs[r * dkp + d], s[r]);
			}
			const int b = bucket ? bucket[i - j] : 0;
#pragma unroll
			for (int r = 0; r < R; ++r)
				if (r < nh) p[r] = sigmoidf_(s[r] + (rel ? rel[(size_t)b * n_heads + h0 + r] : 0.f) + bias_h[r]);
		}
		constexpr int KU = 8;
		for (int k0 = 0; k0 < cnt; k0 += KU) {
			float vv[KU][DVC];
#pragma unroll
			for (int u = 0; u < KU; ++u) {
				const int kk = min(k0 + u, cnt - 1); // past the end: a repeated row whose weight is zero
				const int jj = first ? idx0 + kk : lo + idx0 + kk;
				const CT *vr = first ? fbase + (size_t)jj * dk : rbase + (size_t)(jj % ring) * dk;
#pragma unroll
				for (int c = 0; c < DVC; ++c) vv[u][c] = c * 32 + lane < dk ? cache_get(vr, c * 32 + lane) : 0.f;
			}
#pragma unroll
			for (int u = 0; u < KU; ++u)
#pragma unroll
				for (int r = 0; r < R; ++r) {
					const float pk = k0 + u < cnt ? __shfl_sync(kFull, p[r], (k0 + u) & 31) : 0.f;
#pragma unroll
					for (int c = 0; c < DVC; ++c) acc[r][c] = fmaf(pk, vv[u][c], acc[r][c]);
				}
		}
	}
#pragma unroll
	for (int r = 0; r < R; ++r)
#pragma unroll
		for (int c = 0; c < DVC; ++c)
			if (c * 32 + lane < dk) macc[(warp * R + r) * dk + c * 32 + lane] = acc[r][c];
	__syncthreads();
	for (int e = threadIdx.x; e < nh * dk; e += blockDim.x) {
		const int r = e / dk, c = e % dk, h = h0 + r;
		float o = 0.f;
		for (int w = 0; w < kSigWarps; ++w) o += macc[(w * R + r) * dk + c];
		if (part) part[((size_t)(m * n_heads + h) * nsplit + z) * dk + c] = o;
		else out[(size_t)m * ldo + (size_t)h * dk + c] = gate ? o * sigmoidf_(gate[(size_t)m * ldg + (size_t)h * dk + c]) : o;
	}
}
// The same attention for a bf16 ring whose head size is 8, 16, ..., 256: every key row is read as 16-byte pieces by dk / 8
// neighbouring lanes, so that one warp instruction fetches whole rows and eight of them are in flight per lane; each lane
// keeps its 8 channels of the R queries and of the R sums in registers.  The scores of a 32-key tile pass through shared
// memory to the lane = key layout, where the bias is added and the sigmoid taken, and back for the weighted sum, which
// reads the same rows again (the values are the keys).  Same grid, splits, partials and merge as attn_sigmoid_rows_kernel.
template <int R>
__global__ void __launch_bounds__(kSigWarps * 32) attn_sigmoid_lanes_kernel(float *__restrict__ out, int ldo, const float *__restrict__ q, int ldq,
                                                                            const __nv_bfloat16 *__restrict__ ring_buf,
                                                                            const __nv_bfloat16 *__restrict__ first_buf, const float *__restrict__ gate,
                                                                            int ldg, const float *__restrict__ rel, const int *__restrict__ bucket,
                                                                            const float *__restrict__ hb, float *__restrict__ part, int n_heads, int n_kv,
                                                                            int dk, int ring, int window, int keep, float scale, int pos0,
                                                                            const int *__restrict__ ctl) {
	extern __shared__ __align__(16) float sm[];
	float *qs = sm;                              // R x dk
	float *macc = qs + R * dk;                   // kSigWarps x R x dk
	float *sc = macc + kSigWarps * R * dk;       // kSigWarps x R x 32
	const int rep = n_heads / n_kv, hg = (rep + R - 1) / R;
	const int g = blockIdx.x / hg, h0 = g * rep + (blockIdx.x % hg) * R, nh = min(R, g * rep + rep - h0);
	const int m = blockIdx.y, z = blockIdx.z, nsplit = gridDim.z;
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int i = first_pos(ctl, pos0) + m;
	const int lo = window > 0 ? max(0, i - window + 1) : 0;
	const int nfirst = min(keep, lo), ntok = i - lo + 1;
	for (int e = threadIdx.x; e < R * dk; e += blockDim.x) {
		const int r = e / dk, d = e % dk;
		qs[e] = r < nh ? q[(size_t)m * ldq + (size_t)(h0 + r) * dk + d] * scale : 0.f;
	}
	__syncthreads();
	const int LK = dk >> 3, sub = lane % LK, rg = lane / LK, rp = 32 / LK; // piece of the row, row within a step, rows per step
	float qr[R][8], acc[R][8], bias_h[R];
#pragma unroll
	for (int r = 0; r < R; ++r) {
		bias_h[r] = (hb && r < nh) ? hb[h0 + r] : 0.f;
#pragma unroll
		for (int j = 0; j < 8; ++j) qr[r][j] = qs[r * dk + sub * 8 + j], acc[r][j] = 0.f;
	}
	const __nv_bfloat16 *rbase = ring_buf + (size_t)g * ring * dk + sub * 8, *fbase = first_buf ? first_buf + (size_t)g * keep * dk + sub * 8 : nullptr;
	float *scw = sc + warp * R * 32;
	const int ftiles = (nfirst + 31) / 32, ntiles = ftiles + (ntok + 31) / 32, per = (ntiles + nsplit - 1) / nsplit;
	const int t_end = min(ntiles, (z + 1) * per);
	constexpr int KU = 8; // row steps in flight
	for (int t = z * per + warp; t < t_end; t += kSigWarps) {
		const bool first = t < ftiles;
		const int idx0 = first ? t * 32 : (t - ftiles) * 32, cnt = min(32, (first ? nfirst : ntok) - idx0);
		const int j0 = first ? idx0 : lo + idx0; // position of the tile's first key
		auto row_ptr = [&](int row) { // a row past the end repeats the last one; its weight is zero
			const int j = j0 + min(row, cnt - 1);
			return first ? fbase + (size_t)j * dk : rbase + (size_t)(j % ring) * dk;
		};
		// ---- scores ----
		for (int u0 = 0; u0 * rp < cnt; u0 += KU) {
			uint4 w[KU];
#pragma unroll
			for (int u = 0; u < KU; ++u) w[u] = __ldg(reinterpret_cast<const uint4 *>(row_ptr((u0 + u) * rp + rg)));
#pragma unroll
			for (int u = 0; u < KU; ++u) {
				float kf[8], d[R];
				Elem<YALM_BF16>::unpack(w[u], kf);
				const int row = (u0 + u) * rp + rg;
#pragma unroll
				for (int r = 0; r < R; ++r) {
					d[r] = 0.f;
#pragma unroll
					for (int j = 0; j < 8; ++j) d[r] = fmaf(kf[j], qr[r][j], d[r]);
				}
				for (int o = LK >> 1; o > 0; o >>= 1)
#pragma unroll
					for (int r = 0; r < R; ++r) d[r] += __shfl_xor_sync(kFull, d[r], o);
				if (sub == 0 && row < 32) {
#pragma unroll
					for (int r = 0; r < R; ++r) scw[r * 32 + row] = d[r];
				}
			}
		}
		__syncwarp();
		// ---- weights, lane = key ----
		{
			const int b = (bucket && lane < cnt) ? bucket[i - (j0 + lane)] : 0;
#pragma unroll
			for (int r = 0; r < R; ++r) {
				float pv = 0.f;
				if (lane < cnt && r < nh) pv = sigmoidf_(scw[r * 32 + lane] + (rel ? rel[(size_t)b * n_heads + h0 + r] : 0.f) + bias_h[r]);
				scw[r * 32 + lane] = pv;
			}
		}
		__syncwarp();
		// ---- weighted sum of the same rows ----
		for (int u0 = 0; u0 * rp < cnt; u0 += KU) {
			uint4 w[KU];
#pragma unroll
			for (int u = 0; u < KU; ++u) w[u] = __ldg(reinterpret_cast<const uint4 *>(row_ptr((u0 + u) * rp + rg)));
#pragma unroll
			for (int u = 0; u < KU; ++u) {
				float vf[8];
				Elem<YALM_BF16>::unpack(w[u], vf);
				const int row = (u0 + u) * rp + rg;
#pragma unroll
				for (int r = 0; r < R; ++r) {
					const float pk = row < cnt ? scw[r * 32 + row] : 0.f;
#pragma unroll
					for (int j = 0; j < 8; ++j) acc[r][j] = fmaf(pk, vf[j], acc[r][j]);
				}
			}
		}
		__syncwarp(); // the next tile's scores overwrite scw
	}
	// the row groups of a warp hold partial sums of the same channels
	for (int o = 16; o >= LK; o >>= 1)
#pragma unroll
		for (int r = 0; r < R; ++r)
#pragma unroll
			for (int j = 0; j < 8; ++j) acc[r][j] += __shfl_xor_sync(kFull, acc[r][j], o);
	if (rg == 0) {
#pragma unroll
		for (int r = 0; r < R; ++r)
#pragma unroll
			for (int j = 0; j < 8; ++j) macc[(warp * R + r) * dk + sub * 8 + j] = acc[r][j];
	}
	__syncthreads();
	for (int e = threadIdx.x; e < nh * dk; e += blockDim.x) {
		const int r = e / dk, c = e % dk, h = h0 + r;
		float o = 0.f;
		for (int w = 0; w < kSigWarps; ++w) o += macc[(w * R + r) * dk + c];
		if (part) part[((size_t)(m * n_heads + h) * nsplit + z) * dk + c] = o;
		else out[(size_t)m * ldo + (size_t)h * dk + c] = gate ? o * sigmoidf_(gate[(size_t)m * ldg + (size_t)h * dk + c]) : o;
	}
}
__global__ void attn_sigmoid_merge_kernel(float *__restrict__ out, int ldo, const float *__restrict__ part, const float *__restrict__ gate, int ldg,
                                          int n_heads, int dk, int nsplit) {
	const int h = blockIdx.x, m = blockIdx.y;
	const float *pr = part + (size_t)(m * n_heads + h) * nsplit * dk;
	for (int c = threadIdx.x; c < dk; c += blockDim.x) {
		float o = 0.f;
		for (int z = 0; z < nsplit; ++z) o += pr[(size_t)z * dk + c];
		out[(size_t)m * ldo + (size_t)h * dk + c] = gate ? o * sigmoidf_(gate[(size_t)m * ldg + (size_t)h * dk + c]) : o;
	}
}

// ---- x += a (+ b) + sum_j y_j -------------------------------------------------------------------------------------------------
__global__ void residual_sum_rows_kernel(float *__restrict__ x, const float *__restrict__ a, const float *__restrict__ b, const float *__restrict__ y,
                                         int ldy, int nsum, int dim) {
	const int m = blockIdx.y, e = blockIdx.x * blockDim.x + threadIdx.x;
	if (e >= dim) return;
	float v = a ? a[(size_t)m * dim + e] : 0.f;
	if (b) v += b[(size_t)m * dim + e];
	float f = 0.f;
	for (int j = 0; j < nsum; ++j) f += y[((size_t)m * nsum + j) * ldy + e];
	x[(size_t)m * dim + e] += v + f;
}

__global__ void softcap_rows_kernel(float *__restrict__ z, size_t count, float cap) {
	const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (i < count) z[i] = cap * tanhf(z[i] / cap);
}

} // namespace stack
} // namespace yalm

using namespace yalm;
using namespace yalm::stack;

extern "C" int yalm_norm_shift_rows(float *h, float *hs, const float *x, const float *w, int scalar_weight, float w_offset, float eps, const float *shift,
                                    float *state, int n, int dim, int pos0, const int *ctl, yalm_stream_t s) {
	if (!h || !x || !w || n < 1 || dim < 1 || (hs && (!shift || !state || h == x))) return YALM_EINVAL;
	cudaStream_t st = (cudaStream_t)s;
	norm_shift_rows_kernel<<<n, 256, 0, st>>>(h, hs, x, w, scalar_weight, w_offset, eps, shift, state, n == 1, dim, pos0, ctl);
	if (hs && n > 1) return (int)cudaMemcpyAsync(state, h + (size_t)(n - 1) * dim, sizeof(float) * dim, cudaMemcpyDeviceToDevice, st);
	return (int)cudaGetLastError();
}

extern "C" int yalm_conv_act_rows(float *out, int ldo, const float *in, int ldi, const float *w, const float *bias, float *state, int n, int channels,
                                  int taps, int pos0, const int *ctl, yalm_stream_t s) {
	if (!out || !in || !w || (!state && taps > 1) || n < 1 || channels < 1 || taps < 1 || out == in) return YALM_EINVAL;
	cudaStream_t st = (cudaStream_t)s;
	const dim3 grid((channels + 127) / 128, (n + kConvRows - 1) / kConvRows);
	conv_act_rows_kernel<<<grid, 128, 0, st>>>(out, ldo, in, ldi, w, bias, state, n, channels, taps, pos0, ctl);
	if (grid.y > 1 && taps > 1) conv_state_rows_kernel<<<grid.x, 128, 0, st>>>(in, ldi, state, n, channels, taps, pos0, ctl);
	return (int)cudaGetLastError();
}

// See ScanArgs.  k, q: (n, kv heads * D) with head h reading kv head h / rep; v, out: (n, H * P); decay: (n, H) or, with
// decay_per_channel, (n, H * D); vscale, beta: (n, H) or null; skip: (H) or null; state: (H, P, D) fp32.  D <= 256.
extern "C" int yalm_state_scan_rows(float *out, int ldo, const float *k, int ldk, const float *q, int ldq, const float *v, int ldv, const float *decay,
                                    int ldd, int decay_per_channel, const float *vscale, int ldvs, const float *beta, int ldb, const float *skip,
                                    float *state, int n, int heads, int rep, int D, int P, int pos0, const int *ctl, yalm_stream_t s) {
	if (!out || !k || !q || !v || !decay || !state || n < 1 || heads < 1 || rep < 1 || heads % rep || D < 1 || D > kScanMaxD || P < 1) return YALM_EINVAL;
	auto al = [](const float *p, int ld) { return ((uintptr_t)p & 15) == 0 && ld % 4 == 0; };
	const int vec = D % 4 == 0 && al(k, ldk) && al(q, ldq) && (!decay_per_channel || al(decay, ldd));
	ScanArgs a{out, ldo, k, q, v, decay, vscale, beta, skip, ldk, ldq, ldv, ldd, ldvs, ldb, decay_per_channel, state, n, heads, rep, D, P, pos0, ctl, vec};
	const dim3 grid((P + kScanCols - 1) / kScanCols, heads);
	cudaStream_t st = (cudaStream_t)s;
#define SCAN_CASE(EPL_)                                                                                                                      \
	{                                                                                                                                        \
		constexpr size_t smem = sizeof(float) * 2 * ScanLayout<EPL_>::STAGE;                                                                 \
		static bool configured = false;                                                                                                      \
		if (smem > 48 * 1024 && !configured) {                                                                                               \
			YALM_TRY(cudaFuncSetAttribute(state_scan_kernel<EPL_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                 \
			configured = true;                                                                                                               \
		}                                                                                                                                    \
		state_scan_kernel<EPL_><<<grid, kScanCols * 8, smem, st>>>(a);                                                                       \
	}
	if (D <= 8) SCAN_CASE(1)
	else if (D <= 16) SCAN_CASE(2)
	else if (D <= 32) SCAN_CASE(4)
	else if (D <= 64) SCAN_CASE(8)
	else if (D <= 128) SCAN_CASE(16)
	else SCAN_CASE(32)
#undef SCAN_CASE
	return (int)cudaGetLastError();
}

extern "C" int yalm_ssm_prep_rows(float *dt, int lddt, float *decay, int ldd, const float *dt_bias, const float *a_log, int n, int heads, yalm_stream_t s) {
	if (!dt || !decay || !dt_bias || !a_log || n < 1 || heads < 1) return YALM_EINVAL;
	ssm_prep_rows_kernel<<<n, 128, 0, (cudaStream_t)s>>>(dt, lddt, decay, ldd, dt_bias, a_log, heads);
	return (int)cudaGetLastError();
}

extern "C" int yalm_delta_prep_rows(float *q, float *k, int ldqk, float *beta, int ldb, float *g, int ldg, const float *a_log, const float *dt_bias, int n,
                                    int heads, int kv_heads, int dim, float unit_eps, float q_scale, yalm_stream_t s) {
	if (!q || !k || !beta || !g || !a_log || !dt_bias || n < 1 || heads < 1 || kv_heads < 1 || dim < 1) return YALM_EINVAL;
	delta_prep_rows_kernel<<<n, 256, 0, (cudaStream_t)s>>>(q, k, ldqk, beta, ldb, g, ldg, a_log, dt_bias, heads, kv_heads, dim, unit_eps, q_scale);
	return (int)cudaGetLastError();
}

extern "C" int yalm_gated_group_norm_rows(float *out, int ldo, const float *y, int ldy, const float *z, int ldz, const float *w, int n, int dim, int parts,
                                          float eps, yalm_stream_t s) {
	if (!out || !y || !z || !w || n < 1 || parts < 1 || dim < parts || dim % parts) return YALM_EINVAL;
	// few rows (decoding): the part's channels spread over more threads
	const int threads = n * parts < 64 ? std::min(1024, std::max(256, (dim / parts + 127) / 128 * 32)) : 256;
	gated_group_norm_rows_kernel<<<dim3(n, parts), threads, 0, (cudaStream_t)s>>>(out, ldo, y, ldy, z, ldz, w, dim / parts, eps);
	return (int)cudaGetLastError();
}

extern "C" int yalm_head_norm_gate_rows(float *out, int ldo, const float *o, int ldi, const float *gate, int ldg, const float *w, int n, int heads, int vdim,
                                        float eps, yalm_stream_t s) {
	return yalm_head_norm_act_rows(out, ldo, o, ldi, gate, ldg, w, n, heads, vdim, eps, 0, s);
}

// gate_silu != 0: the gate is silu(gate) instead of sigmoid(gate)
extern "C" int yalm_head_norm_act_rows(float *out, int ldo, const float *o, int ldi, const float *gate, int ldg, const float *w, int n, int heads, int vdim,
                                       float eps, int gate_silu, yalm_stream_t s) {
	if (!out || !o || !gate || !w || n < 1 || heads < 1 || vdim < 1) return YALM_EINVAL;
	head_norm_gate_rows_kernel<<<dim3((heads + 3) / 4, n), 128, 0, (cudaStream_t)s>>>(out, ldo, o, ldi, gate, ldg, w, heads, vdim, eps, gate_silu);
	return (int)cudaGetLastError();
}

extern "C" int yalm_qk_bias_append_rows(float *q, float *k, int ld, const float *qb, const float *kb, void *ring_buf, void *first_buf, int n, int n_heads,
                                        int n_kv, int dk, int ring, int keep, int cache_f32, int pos0, const int *ctl, yalm_stream_t s) {
	if (!q || !k || !ring_buf || n < 1 || ring < 1 || keep < 0 || (keep > 0 && !first_buf)) return YALM_EINVAL;
	cudaStream_t st = (cudaStream_t)s;
	if (cache_f32)
		qk_bias_append_rows_kernel<float><<<n, 256, 0, st>>>(q, k, ld, qb, kb, (float *)ring_buf, (float *)first_buf, n_heads * dk, n_kv * dk, dk, ring, keep,
		                                                     pos0, ctl);
	else
		qk_bias_append_rows_kernel<__nv_bfloat16><<<n, 256, 0, st>>>(q, k, ld, qb, kb, (__nv_bfloat16 *)ring_buf, (__nv_bfloat16 *)first_buf, n_heads * dk,
		                                                             n_kv * dk, dk, ring, keep, pos0, ctl);
	return (int)cudaGetLastError();
}

constexpr int kSigMaxParts = 4096; // (row, head, split) partial sums the workspace holds
extern "C" size_t yalm_attn_sigmoid_workspace(int dk) {
	return (size_t)kSigMaxParts * dk;
}

template <typename CT, int R, int DVC>
static int launch_attn_sigmoid(float *out, int ldo, const float *q, int ldq, const void *ring_buf, const void *first_buf, const float *gate, int ldg,
                               const float *rel, const int *bucket, const float *hb, float *ws, int n, int n_heads, int n_kv, int dk, int ring, int window,
                               int keep, float scale, int nsplit, int pos0, const int *ctl, cudaStream_t st) {
	const int rep = n_heads / n_kv, hg = (rep + R - 1) / R;
	const size_t smem = sizeof(float) * ((size_t)R * ((dk + 3) & ~3) + (size_t)kSigWarps * R * dk);
	if (smem > 48 * 1024) return YALM_EINVAL;
	attn_sigmoid_rows_kernel<CT, R, DVC><<<dim3(n_kv * hg, n, nsplit), kSigWarps * 32, smem, st>>>(
	    out, ldo, q, ldq, (const CT *)ring_buf, (const CT *)first_buf, gate, ldg, rel, bucket, hb, nsplit > 1 ? ws : nullptr, n_heads, n_kv, dk, ring, window,
	    keep, scale, pos0, ctl);
	if (nsplit > 1) attn_sigmoid_merge_kernel<<<dim3(n_heads, n), 128, 0, st>>>(out, ldo, ws, gate, ldg, n_heads, dk, nsplit);
	return (int)cudaGetLastError();
}

template <int R>
static int launch_attn_sigmoid_lanes(float *out, int ldo, const float *q, int ldq, const void *ring_buf, const void *first_buf, const float *gate, int ldg,
                                     const float *rel, const int *bucket, const float *hb, float *ws, int n, int n_heads, int n_kv, int dk, int ring,
                                     int window, int keep, float scale, int nsplit, int pos0, const int *ctl, cudaStream_t st) {
	const int rep = n_heads / n_kv, hg = (rep + R - 1) / R;
	const size_t smem = sizeof(float) * ((size_t)R * dk + (size_t)kSigWarps * R * dk + kSigWarps * R * 32);
	if (smem > 48 * 1024) return YALM_EINVAL;
	attn_sigmoid_lanes_kernel<R><<<dim3(n_kv * hg, n, nsplit), kSigWarps * 32, smem, st>>>(
	    out, ldo, q, ldq, (const __nv_bfloat16 *)ring_buf, (const __nv_bfloat16 *)first_buf, gate, ldg, rel, bucket, hb, nsplit > 1 ? ws : nullptr, n_heads, n_kv,
	    dk, ring, window, keep, scale, pos0, ctl);
	if (nsplit > 1) attn_sigmoid_merge_kernel<<<dim3(n_heads, n), 128, 0, st>>>(out, ldo, ws, gate, ldg, n_heads, dk, nsplit);
	return (int)cudaGetLastError();
}

// rel: (rows, n_heads) fp32 with bucket[distance] naming the row, or null; hb: (n_heads) or null; gate: (n, n_heads * dk)
// raw gate values with row stride ldg, or null.  workspace: yalm_attn_sigmoid_workspace(dk) floats or null (never split);
// context: the most positions a sequence reaches.
extern "C" int yalm_attn_sigmoid_rows(float *out, int ldo, const float *q, int ldq, const void *ring_buf, const void *first_buf, const float *gate, int ldg,
                                      const float *rel, const int *bucket, const float *hb, float *workspace, int n, int n_heads, int n_kv, int dk, int ring,
                                      int window, int keep, float scale, int cache_f32, int context, int pos0, const int *ctl, yalm_stream_t s) {
	if (!out || !q || !ring_buf || n < 1 || n_kv < 1 || n_heads % n_kv || dk < 1 || dk > 256 || (keep > 0 && !first_buf) || (rel && !bucket)) return YALM_EINVAL;
	cudaStream_t st = (cudaStream_t)s;
	const int rep = n_heads / n_kv, R = rep >= 2 ? 4 : 1, hg = (rep + R - 1) / R;
	int nsplit = 1;
	const int ctas = n_kv * hg * n;
	if (workspace && ctas < 296) { // few CTAs (decoding): split the keys; the count depends on shapes only, never on the position
		const int most_keys = window > 0 ? window + keep : (context > 0 ? context : ring);
		const int tiles = (most_keys + 31) / 32 + 1;
		nsplit = std::min({(296 + ctas - 1) / ctas, std::max(1, (tiles + kSigWarps - 1) / kSigWarps), std::max(1, kSigMaxParts / (n * n_heads)), 64});
	}
	// bf16 ring, head sizes 8 * 2^k: rows read as 16-byte pieces by lane groups.  Heads per CTA: four share every key read; with
	// few CTAs (decoding) fewer heads per CTA spread the same work over more SMs.  YALM_STACK_ATTN_LANES=0: the lane-per-key kernel.
	static const bool lanes_off = [] { const char *e = getenv("YALM_STACK_ATTN_LANES"); return e && e[0] == '0'; }();
	if (!cache_f32 && dk >= 8 && (dk & (dk - 1)) == 0 && aligned16(ring_buf) && aligned16(first_buf) && !lanes_off) {
		int RL = R;
		while (RL > 1 && (long)n_kv * ((rep + RL - 1) / RL) * n * nsplit < device_info().sms) RL >>= 1;
#define SIG_LANES(R_)                                                                                                                             \
	return launch_attn_sigmoid_lanes<R_>(out, ldo, q, ldq, ring_buf, first_buf, gate, ldg, rel, bucket, hb, workspace, n, n_heads, n_kv, dk, ring, window, \
	                                     keep, scale, nsplit, pos0, ctl, st)
		if (RL == 1) SIG_LANES(1);
		if (RL == 2) SIG_LANES(2);
		SIG_LANES(4);
#undef SIG_LANES
	}
#define SIG_CASE(CT, R_, DVC_)                                                                                                                     \
	return launch_attn_sigmoid<CT, R_, DVC_>(out, ldo, q, ldq, ring_buf, first_buf, gate, ldg, rel, bucket, hb, workspace, n, n_heads, n_kv, dk, ring, \
	                                         window, keep, scale, nsplit, pos0, ctl, st)
#define SIG_DVC(CT, R_)                                                                                                                            \
	if (dk <= 64) SIG_CASE(CT, R_, 2);                                                                                                             \
	else if (dk <= 128) SIG_CASE(CT, R_, 4);                                                                                                       \
	else SIG_CASE(CT, R_, 8)
	if (cache_f32) {
		if (R == 1) { SIG_DVC(float, 1); }
		else { SIG_DVC(float, 4); }
	} else {
		if (R == 1) { SIG_DVC(__nv_bfloat16, 1); }
		else { SIG_DVC(__nv_bfloat16, 4); }
	}
#undef SIG_DVC
#undef SIG_CASE
}

extern "C" int yalm_residual_sum_rows(float *x, const float *a, const float *b, const float *y, int ldy, int nsum, int n, int dim, yalm_stream_t s) {
	if (!x || n < 1 || dim < 1 || nsum < 0 || (nsum && !y)) return YALM_EINVAL;
	residual_sum_rows_kernel<<<dim3((dim + 255) / 256, n), 256, 0, (cudaStream_t)s>>>(x, a, b, y, ldy, nsum, dim);
	return (int)cudaGetLastError();
}

extern "C" int yalm_softcap_rows(float *z, int n, int dim, float cap, yalm_stream_t s) {
	if (!z || n < 1 || dim < 1 || !(cap > 0.f)) return YALM_EINVAL;
	const size_t count = (size_t)n * dim;
	softcap_rows_kernel<<<(unsigned)((count + 255) / 256), 256, 0, (cudaStream_t)s>>>(z, count, cap);
	return (int)cudaGetLastError();
}
