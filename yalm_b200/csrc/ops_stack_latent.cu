// Row ops of pre-norm layers with an input convolution, latent attention and gated linear attention (stack.cpp).  Like the other
// row ops every kernel takes n rows = n consecutive positions of one sequence (n = 1: a decode step), fp32 activations, and
// positions from the argument or the device control block.  A call whose first position is 0 starts a sequence: stored state
// is taken as zero.
//
//   norm_conv_rows        h = norm(x) w (layer norm without bias, or RMS), u = h + conv(h): a causal convolution over time on each
//                         channel; the last taps - 1 rows of h are sequence state
//   latent_post_rows      the packed projection of a latent-attention layer: the query latent RMS-normed in place; the key / value
//                         latent RMS-normed and, beside the rotated shared key part, written to the cache row of its position
//   latent_query_rows     per head: the unrotated query part multiplied through W_uk onto the latent's coordinates, the rotated part
//                         turned by its position: the query against cached rows [latent | rotated key part]
//   head_linear_gate_rows per head out = W_h x_h (the attention's sum over latents through W_uv), times sigmoid(gate)
//   gla_prep_rows         decays a = sigmoid(z + b)^(1 / tau) and the query scale of gated linear attention
//   depth_average_rows    keeps a layer's result and forms the weighted sum of all results so far
//   layer_norm_gather_rows  final layer norm of the rows whose logits are wanted
#include "common.cuh"

#include <cuda_bf16.h>

#include <algorithm>

#include "launch.h"
#include "stack_rows.cuh"

namespace yalm {
namespace stack {

// ---- norm + input convolution -------------------------------------------------------------------------------------------
// Row `row` of the call (negative: a position before the call, read from the state; before the sequence: zero) normed into
// dst (dim floats of shared memory).  Two passes for the layer norm: mean, then the mean of the squared deviations.  The row
// goes to shared memory first, with its loads unrolled so that several are in flight per thread: with one CTA per row (and one
// row per decode step) the memory latency of every dependent pass is the kernel's time.
__device__ __forceinline__ void normed_row(float *dst, const float *x, const float *__restrict__ w, const float *state, int row, int p0, int taps, int dim,
                                           int layer_norm, float eps, float *red) {
	if (row < 0) {
		const bool have = p0 + row >= 0;
		const float *src = state + (size_t)(taps - 1 + row) * dim;
#pragma unroll 8
		for (int e = threadIdx.x; e < dim; e += blockDim.x) dst[e] = have ? src[e] : 0.f;
		return;
	}
	const float *src = x + (size_t)row * dim;
	float s = 0.f;
#pragma unroll 8
	for (int e = threadIdx.x; e < dim; e += blockDim.x) {
		const float v = src[e];
		dst[e] = v;
		s += v;
	}
	const float mean = layer_norm ? block_sum(s, red) / dim : 0.f;
	float ss = 0.f;
#pragma unroll 8
	for (int e = threadIdx.x; e < dim; e += blockDim.x) {
		const float d = dst[e] - mean;
		ss += d * d;
	}
	ss = block_sum(ss, red);
	const float r = 1.0f / sqrtf(ss / dim + eps);
#pragma unroll 8
	for (int e = threadIdx.x; e < dim; e += blockDim.x) dst[e] = (dst[e] - mean) * r * w[e];
}

// One CTA per row m: the normed rows m - taps + 1 .. m are rebuilt in shared memory (rows of the call from x, earlier ones from
// the state (taps - 1, dim), whose slot s is the normed input of position p0 - (taps - 1) + s), u = h_m + sum_j cw[:, j] h_(m-taps+1+j).
// h_m also goes to h.  single != 0 (one-row calls): the CTA then shifts the state itself.
__global__ void __launch_bounds__(256) norm_conv_rows_kernel(float *__restrict__ u, float *__restrict__ h, const float *x, const float *__restrict__ w,
                                                             int layer_norm, float eps, const float *__restrict__ cw, float *state, int dim, int taps,
                                                             int single, int pos0, const int *__restrict__ ctl, float *xadd, const float *__restrict__ add) {
	extern __shared__ float hs[]; // taps x dim
	__shared__ float red[33];
	const int m = blockIdx.x, p0 = first_pos(ctl, pos0);
	if (add) { // one-row calls: the residual takes the previous sublayer's output first
#pragma unroll 8
		for (int e = threadIdx.x; e < dim; e += blockDim.x) xadd[e] += add[e];
		__syncthreads();
	}
	for (int j = 0; j < taps; ++j) normed_row(hs + (size_t)j * dim, x, w, state, m - (taps - 1) + j, p0, taps, dim, layer_norm, eps, red);
	__syncthreads();
#pragma unroll 4
	for (int e = threadIdx.x; e < dim; e += blockDim.x) {
		const float hm = hs[(size_t)(taps - 1) * dim + e];
		float acc = hm;
		for (int j = 0; j < taps; ++j) acc = fmaf(cw[(size_t)e * taps + j], hs[(size_t)j * dim + e], acc);
		u[(size_t)m * dim + e] = acc;
		h[(size_t)m * dim + e] = hm;
		if (single)
			for (int s = 0; s < taps - 1; ++s) state[(size_t)s * dim + e] = hs[(size_t)(s + 1) * dim + e];
	}
}
// One-row calls (a decode step): every thread fetches its channels of x (+ add), the norm weight, the stored rows and the
// convolution weights at once, so that the whole kernel is one memory round trip, two block sums and the stores.  EPT channels
// per thread, at most kOneTaps taps.
constexpr int kOneTaps = 5, kOneThreads = 1024;
template <int EPT>
__global__ void __launch_bounds__(kOneThreads) norm_conv_one_kernel(float *__restrict__ u, float *__restrict__ h, float *x, const float *__restrict__ add,
                                                                    const float *__restrict__ w, int layer_norm, float eps, const float *__restrict__ cw,
                                                                    float *state, int dim, int taps, int pos0, const int *__restrict__ ctl) {
	__shared__ float red[33];
	const int p0 = first_pos(ctl, pos0);
	float xv[EPT], wv[EPT], sv[kOneTaps - 1][EPT], cv[kOneTaps][EPT];
#pragma unroll
	for (int i = 0; i < EPT; ++i) {
		const int e = threadIdx.x + i * kOneThreads;
		const bool in = e < dim;
		xv[i] = in ? x[e] : 0.f;
		if (add && in) xv[i] += add[e];
		wv[i] = in ? w[e] : 0.f;
#pragma unroll
		for (int s = 0; s < kOneTaps - 1; ++s) sv[s][i] = (in && s < taps - 1 && p0 - (taps - 1) + s >= 0) ? state[(size_t)s * dim + e] : 0.f;
#pragma unroll
		for (int j = 0; j < kOneTaps; ++j) cv[j][i] = (in && j < taps) ? cw[(size_t)e * taps + j] : 0.f;
	}
	float s1 = 0.f;
#pragma unroll
	for (int i = 0; i < EPT; ++i) s1 += xv[i];
	const float mean = layer_norm ? block_sum(s1, red) / dim : 0.f;
	float ss = 0.f;
#pragma unroll
	for (int i = 0; i < EPT; ++i) {
		const float d = threadIdx.x + i * kOneThreads < dim ? xv[i] - mean : 0.f;
		ss += d * d;
	}
	ss = block_sum(ss, red);
	const float r = 1.0f / sqrtf(ss / dim + eps);
#pragma unroll
	for (int i = 0; i < EPT; ++i) {
		const int e = threadIdx.x + i * kOneThreads;
		if (e >= dim) continue;
		const float hm = (xv[i] - mean) * r * wv[i];
		float acc = hm;
#pragma unroll
		for (int j = 0; j < kOneTaps; ++j)
			if (j < taps) acc = fmaf(cv[j][i], j == taps - 1 ? hm : sv[j][i], acc);
		u[e] = acc, h[e] = hm;
		if (add) x[e] = xv[i];
#pragma unroll
		for (int s = 0; s < kOneTaps - 1; ++s)
			if (s < taps - 1) state[(size_t)s * dim + e] = s + 1 == taps - 1 ? hm : sv[s + 1][i];
	}
}

// After a call of n > 1 rows: slot s <- the normed input of row n - (taps - 1) + s (from h, or an old slot above s).
__global__ void norm_conv_state_kernel(float *state, const float *__restrict__ h, int n, int dim, int taps, int pos0, const int *__restrict__ ctl) {
	const int e = blockIdx.x * blockDim.x + threadIdx.x, p0 = first_pos(ctl, pos0);
	if (e >= dim) return;
	for (int s = 0; s < taps - 1; ++s) {
		const int row = n - (taps - 1) + s;
		state[(size_t)s * dim + e] = row >= 0 ? h[(size_t)row * dim + e] : (p0 + row >= 0 ? state[(size_t)(taps - 1 + row) * dim + e] : 0.f);
	}
}

// ---- rotary positions ---------------------------------------------------------------------------------------------------
// Pair i of a vector at position p turns by p * freq[i]; cos and sin carry the magnitude factor.  Position, angle and the
// rotation are fp32.  interleaved: the pair is (2 i, 2 i + 1), else (i, i + half).
__device__ __forceinline__ void rotate_pair(float a, float b, int p, float freq, float mag, float *ra, float *rb) {
	const float ang = (float)p * freq;
	float sn, cs;
	sincosf(ang, &sn, &cs);
	sn *= mag, cs *= mag;
	*ra = a * cs - b * sn, *rb = b * cs + a * sn;
}

// ---- latent attention: norms, rotation, cache append ----------------------------------------------------------------------
// Row m of the packed projection P (ld): [o_q, +q_rank) the query latent: RMS norm with weight qw in place.  With a cache of
// its own, [o_kv, +kv_rank) RMS-normed with weight kw is the key / value latent and [o_kv + kv_rank, +rot_dim) the shared key
// part, whose first rot_dims channels are rotated; both go to the ring row (slot p % ring) as [latent | key part].
template <typename CT>
__global__ void __launch_bounds__(256) latent_post_rows_kernel(float *__restrict__ P, int ld, int o_q, int q_rank, const float *__restrict__ qw, int o_kv,
                                                               int kv_rank, int rot_dim, const float *__restrict__ kw, CT *__restrict__ ring_buf, int ring,
                                                               const float *__restrict__ freq, float mag, int rot_dims, int interleaved, float eps,
                                                               int pos0, const int *__restrict__ ctl) {
	__shared__ float red[33];
	const int m = blockIdx.x, p = first_pos(ctl, pos0) + m;
	float *row = P + (size_t)m * ld;
	if (q_rank > 0) { // 0: the queries are projected at full rank, there is no query latent
		float ss = 0.f;
		for (int e = threadIdx.x; e < q_rank; e += blockDim.x) ss += row[o_q + e] * row[o_q + e];
		ss = block_sum(ss, red);
		const float r = 1.0f / sqrtf(ss / q_rank + eps);
		for (int e = threadIdx.x; e < q_rank; e += blockDim.x) row[o_q + e] = row[o_q + e] * r * qw[e];
	}
	if (!ring_buf) return;
	float ss = 0.f;
	for (int e = threadIdx.x; e < kv_rank; e += blockDim.x) ss += row[o_kv + e] * row[o_kv + e];
	ss = block_sum(ss, red);
	const float r = 1.0f / sqrtf(ss / kv_rank + eps);
	CT *dst = ring_buf + (size_t)(p % ring) * (kv_rank + rot_dim);
	for (int e = threadIdx.x; e < kv_rank; e += blockDim.x) cache_put(dst, e, row[o_kv + e] * r * kw[e]);
	const float *kr = row + o_kv + kv_rank;
	const int half = rot_dims / 2;
	for (int i = threadIdx.x; i < half; i += blockDim.x) {
		const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
		float a, b;
		rotate_pair(kr[ia], kr[ib], p, freq[i], mag, &a, &b);
		cache_put(dst, kv_rank + ia, a), cache_put(dst, kv_rank + ib, b);
	}
	for (int e = rot_dims + threadIdx.x; e < rot_dim; e += blockDim.x) cache_put(dst, kv_rank + e, kr[e]);
}

// ---- latent attention: the query against cached rows ------------------------------------------------------------------------
// q (n, heads (dim + rot_dim)), per head [unrotated | rotated].  out (n, heads (kv_rank + rot_dim)):
//   out[m, h, c] = sum_d q[m, h, d] ukt[h, c, d]   (c < kv_rank; ukt (heads, kv_rank, dim): every head's W_uk transposed)
//   out[m, h, kv_rank + j] = the rotated part turned by position p0 + m
// so that out[m, h] . [latent_j | key part_j] is the score of head h against position j.  One CTA per (head, block of RB rows);
// a thread owns output channels c and walks d with the rows' queries in shared memory: neighbouring threads read neighbouring
// weights.
constexpr int kLqRows = 8;
template <int DT>
__global__ void __launch_bounds__(64) latent_query_rows_kernel(float *__restrict__ out, int ldo, const float *__restrict__ q, int ldq,
                                                                const void *__restrict__ ukt, int n, int dim, int rot_dim, int kv_rank,
                                                                const float *__restrict__ freq, float mag, int rot_dims, int interleaved, int pos0,
                                                                const int *__restrict__ ctl) {
	extern __shared__ float qs[]; // kLqRows x (dim + rot_dim)
	const int h = blockIdx.x, m0 = blockIdx.y * kLqRows, mb = min(kLqRows, n - m0), dq = dim + rot_dim, p0 = first_pos(ctl, pos0);
#pragma unroll 4
	for (int e = threadIdx.x; e < kLqRows * dq; e += blockDim.x) {
		const int i = e / dq, d = e % dq;
		qs[e] = i < mb ? q[(size_t)(m0 + i) * ldq + (size_t)h * dq + d] : 0.f;
	}
	__syncthreads();
	const size_t obase = (size_t)h * (kv_rank + rot_dim);
	// grid.z cuts the output channels into pieces of one per thread: a decode row then still fills the GPU.  The weights are
	// stored transposed, (heads, kv_rank, dim): an output channel's weights are one contiguous row, fetched as 16-byte pieces
	// that are all in flight at once.
	const bool vec = dim % Elem<DT>::VEC == 0 && aligned16(ukt) && dim <= 16 * Elem<DT>::VEC;
	for (int c = blockIdx.z * blockDim.x + threadIdx.x; c < kv_rank; c += gridDim.z * blockDim.x) {
		float acc[kLqRows];
#pragma unroll
		for (int i = 0; i < kLqRows; ++i) acc[i] = 0.f;
		const size_t roff = ((size_t)h * kv_rank + c) * dim;
		if (vec) {
			using T = typename Elem<DT>::T;
			constexpr int V = Elem<DT>::VEC;
			const T *wr = static_cast<const T *>(ukt) + roff;
			uint4 wv[16];
#pragma unroll
			for (int k = 0; k < 16; ++k)
				if (k * V < dim) wv[k] = __ldg(reinterpret_cast<const uint4 *>(wr + k * V));
#pragma unroll
			for (int k = 0; k < 16; ++k)
				if (k * V < dim) {
					float f[8];
					Elem<DT>::unpack(wv[k], f);
#pragma unroll
					for (int j = 0; j < V; ++j)
#pragma unroll
						for (int i = 0; i < kLqRows; ++i) acc[i] = fmaf(f[j], qs[i * dq + k * V + j], acc[i]);
				}
		} else
			for (int d = 0; d < dim; ++d) {
				const float wv = Elem<DT>::get(ukt, roff + d);
#pragma unroll
				for (int i = 0; i < kLqRows; ++i) acc[i] = fmaf(wv, qs[i * dq + d], acc[i]);
			}
#pragma unroll
		for (int i = 0; i < kLqRows; ++i)
			if (i < mb) out[(size_t)(m0 + i) * ldo + obase + c] = acc[i];
	}
	const int half = rot_dims / 2;
	if (blockIdx.z) return;
	for (int e = threadIdx.x; e < mb * rot_dim; e += blockDim.x) {
		const int i = e / rot_dim, j = e % rot_dim;
		const float *qr = qs + i * dq + dim;
		float *dst = out + (size_t)(m0 + i) * ldo + obase + kv_rank;
		if (j >= rot_dims) dst[j] = qr[j];
		else if (j < half) {
			const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + half;
			rotate_pair(qr[ia], qr[ib], p0 + m0 + i, freq[j], mag, dst + ia, dst + ib);
		}
	}
}

// ---- per-head linear map with a sigmoid gate ----------------------------------------------------------------------------
// out[m, h, j] = (sum_c w[h N + j, c] x[m, h, c]) * sigmoid(gate[m, h, j]) (gate null: no gate); w (heads N, K) row-major.
// One CTA per (head, block of RB rows); a warp owns outputs j, its lanes stride the K inputs (coalesced weight rows), the
// rows' inputs sit in shared memory.
constexpr int kHlRows = 8;
template <int DT>
__global__ void __launch_bounds__(256) head_linear_gate_rows_kernel(float *__restrict__ out, int ldo, const float *__restrict__ x, int ldx,
                                                                    const void *__restrict__ w, const float *__restrict__ gate, int ldg, int n, int N,
                                                                    int K) {
	extern __shared__ __align__(16) float xs[]; // kHlRows x K
	const int h = blockIdx.x, m0 = blockIdx.y * kHlRows, mb = min(kHlRows, n - m0);
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	for (int e = threadIdx.x; e < kHlRows * K; e += blockDim.x) {
		const int i = e / K, c = e % K;
		xs[e] = i < mb ? x[(size_t)(m0 + i) * ldx + (size_t)h * K + c] : 0.f;
	}
	__syncthreads();
	const bool vec = K % Elem<DT>::VEC == 0 && aligned16(w) && ((size_t)K * sizeof(typename Elem<DT>::T)) % 16 == 0;
	if (mb <= 2 && vec) { // decode rows: 16-byte weight loads, several in flight per lane, one row at a time
		for (int j = blockIdx.z * 8 + warp; j < N; j += gridDim.z * 8)
			for (int i = 0; i < mb; ++i) {
				const float v = warp_dot<DT>(w, ((size_t)h * N + j) * K, xs + i * K, K, true);
				if (lane == 0) {
					const size_t o = (size_t)(m0 + i) * ldo + (size_t)h * N + j;
					out[o] = gate ? v / (1.0f + expf(-gate[(size_t)(m0 + i) * ldg + (size_t)h * N + j])) : v;
				}
			}
		return;
	}
	for (int j = blockIdx.z * 8 + warp; j < N; j += gridDim.z * 8) {
		float acc[kHlRows];
#pragma unroll
		for (int i = 0; i < kHlRows; ++i) acc[i] = 0.f;
		const size_t roff = ((size_t)h * N + j) * K;
		for (int c = lane; c < K; c += 32) {
			const float wv = Elem<DT>::get(w, roff + c);
#pragma unroll
			for (int i = 0; i < kHlRows; ++i) acc[i] = fmaf(wv, xs[i * K + c], acc[i]);
		}
#pragma unroll
		for (int i = 0; i < kHlRows; ++i) {
			const float v = warp_sum(acc[i]);
			if (lane == 0 && i < mb) {
				const size_t o = (size_t)(m0 + i) * ldo + (size_t)h * N + j;
				out[o] = gate ? v / (1.0f + expf(-gate[(size_t)(m0 + i) * ldg + (size_t)h * N + j])) : v;
			}
		}
	}
}

// ---- gated linear attention: decays and query scale ---------------------------------------------------------------------------
// z (n, channels) in place: a = sigmoid(z + b)^(1 / tau) = exp(log sigmoid(z + b) / tau), log sigmoid(y) = min(y, 0) - log1p(exp(-|y|));
// q (n, channels, ldq) in place: q *= q_scale.  All fp32.
__global__ void gla_prep_rows_kernel(float *__restrict__ z, int ldz, const float *__restrict__ b, float inv_tau, float *__restrict__ q, int ldq,
                                     float q_scale, int channels) {
	const int m = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
	if (c >= channels) return;
	const float y = z[(size_t)m * ldz + c] + b[c];
	z[(size_t)m * ldz + c] = expf((fminf(y, 0.f) - log1pf(expf(-fabsf(y)))) * inv_tau);
	q[(size_t)m * ldq + c] *= q_scale;
}

// ---- weighted sum over depth ------------------------------------------------------------------------------------------------
// hist holds one (n, dim) slab per result (slab stride `stride` floats): slab count - 1 <- x (+ a (+ b) + sum_j slots[j]: the
// sublayer outputs not yet added); then, with weights w (count), x <- sum_j w[j] slab_j (w null: x keeps the result).
__global__ void depth_average_rows_kernel(float *__restrict__ x, float *__restrict__ hist, size_t stride, const float *__restrict__ w, int count,
                                          size_t total, const float *__restrict__ a, const float *__restrict__ b, const float *__restrict__ y, int ldy,
                                          int nsum, int dim) {
	const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= total) return;
	float v = x[i];
	if (a) v += a[i];
	if (b) v += b[i];
	if (y) {
		const size_t m = i / dim, e = i % dim;
		float sy = 0.f;
		for (int j = 0; j < nsum; ++j) sy += y[(m * nsum + j) * ldy + e];
		v += sy;
	}
	hist[(size_t)(count - 1) * stride + i] = v;
	if (w) {
		float acc = 0.f;
		for (int j = 0; j < count - 1; ++j) acc = fmaf(w[j], hist[(size_t)j * stride + i], acc);
		v = fmaf(w[count - 1], v, acc);
	}
	x[i] = v;
}

// ---- latent attention, prompt portions: keys and values written out per head for the tensor-core attention -------------------
// The cached rows of positions first .. first + count - 1 (bf16 ring, row = [latent | key part], slot = position % ring):
// their latents as one dense bf16 operand (count, kv_rank) ...
__global__ void latent_gather_rows_kernel(__nv_bfloat16 *__restrict__ out, const __nv_bfloat16 *__restrict__ ring_buf, int ring, int row, int kv_rank,
                                          int first) {
	const int j = blockIdx.x;
	const __nv_bfloat16 *src = ring_buf + (size_t)((first + j) % ring) * row;
	for (int e = threadIdx.x; e < kv_rank; e += blockDim.x) out[(size_t)j * kv_rank + e] = src[e];
}
// ... and, from kv (count, heads (dim + vdim)) = latents x [W_uk ; W_uv]^T (fp32: all heads' unrotated keys, then all heads' values),
// per head the key [unrotated | the row's rotated key part] and the value, as bf16 rows of head-major rings (head, slot, channel)
// with slot = position % ring_out: what the windowed tensor-core attention reads.
__global__ void __launch_bounds__(256) latent_pack_rings_kernel(__nv_bfloat16 *__restrict__ kout, __nv_bfloat16 *__restrict__ vout,
                                                                const float *__restrict__ kv, int ldkv, const __nv_bfloat16 *__restrict__ ring_buf,
                                                                int ring, int row, int kv_rank, int rot_dim, int heads, int dim, int vdim, int ring_out,
                                                                int first) {
	const int j = blockIdx.x, p = first + j, dk = dim + rot_dim;
	const float *src = kv + (size_t)j * ldkv;
	const __nv_bfloat16 *kr = ring_buf + (size_t)(p % ring) * row + kv_rank;
	const size_t slot = (size_t)(p % ring_out);
	for (int e = threadIdx.x; e < heads * dk; e += blockDim.x) {
		const int h = e / dk, d = e % dk;
		kout[((size_t)h * ring_out + slot) * dk + d] = d < dim ? __float2bfloat16_rn(src[h * dim + d]) : kr[d - dim];
	}
	for (int e = threadIdx.x; e < heads * vdim; e += blockDim.x) {
		const int h = e / vdim, d = e % vdim;
		vout[((size_t)h * ring_out + slot) * vdim + d] = __float2bfloat16_rn(src[heads * dim + e]);
	}
}
// In place: channels [offset, offset + rot_dims) of every head (head_size channels each) of row m turned by position p0 + m.
__global__ void rotate_heads_rows_kernel(float *__restrict__ q, int ldq, int heads, int head_size, int offset, const float *__restrict__ freq, float mag,
                                         int rot_dims, int interleaved, int pos0, const int *__restrict__ ctl) {
	const int m = blockIdx.x, p = first_pos(ctl, pos0) + m, half = rot_dims / 2;
	for (int e = threadIdx.x; e < heads * half; e += blockDim.x) {
		const int h = e / half, i = e % half;
		float *v = q + (size_t)m * ldq + (size_t)h * head_size + offset;
		const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
		float a, b;
		rotate_pair(v[ia], v[ib], p, freq[i], mag, &a, &b);
		v[ia] = a, v[ib] = b;
	}
}
// x[m, :dim] *= sigmoid(gate[m, :dim])
__global__ void sigmoid_gate_rows_kernel(float *__restrict__ x, int ldx, const float *__restrict__ gate, int ldg, int dim) {
	const int m = blockIdx.y, e = blockIdx.x * blockDim.x + threadIdx.x;
	if (e < dim) x[(size_t)m * ldx + e] /= 1.0f + expf(-gate[(size_t)m * ldg + e]);
}

// ---- latent attention over cached rows, one pass ---------------------------------------------------------------------------------
// Every head reads the same bf16 row [latent | rotated key part] of a position: its key is the whole row (dk channels), its
// value the row's first dv channels.  A warp takes one row at a time as 16-byte pieces (lane l holds pieces l, l + 32, ...: one
// instruction fetches 512 contiguous bytes), so a row is read ONCE for the scores of R heads and for their weighted sums: the
// pieces that made the score are the value.  KB rows are in flight per warp; their scores are reduced with shuffles, one
// online-softmax correction is applied per batch, and the warps of a CTA and the splits of a query merge as in the windowed
// attention (partials: accumulator, max, sum).  grid (head groups, rows, splits).
constexpr int kLaWarps = 4, kLaBatch = 4, kLaMaxParts = 4096;
template <int R, int NP>
__global__ void __launch_bounds__(kLaWarps * 32) attn_latent_rows_kernel(float *__restrict__ out, int ldo, const float *__restrict__ q, int ldq,
                                                                         const __nv_bfloat16 *__restrict__ rows, int ld, float *__restrict__ part,
                                                                         int n_heads, int dk, int dv, int ring, int window, float scale, int pos0,
                                                                         const int *__restrict__ ctl, const float *__restrict__ sink) {
	extern __shared__ __align__(16) float sm[];
	const int dkp = NP * 256;
	float *qs = sm;                               // R x dkp, zero beyond dk
	float *macc = qs + R * dkp;                   // kLaWarps x R x dv
	float *mml = macc + kLaWarps * R * dv;        // kLaWarps x R x 2
	const int h0 = blockIdx.x * R, nh = min(R, n_heads - h0), m = blockIdx.y, z = blockIdx.z, nsplit = gridDim.z;
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int i = first_pos(ctl, pos0) + m, lo = window > 0 ? max(0, i - window + 1) : 0, ntok = i - lo + 1;
#pragma unroll 8
	for (int e = threadIdx.x; e < R * dkp; e += blockDim.x) {
		const int r = e / dkp, d = e % dkp;
		qs[e] = (r < nh && d < dk) ? q[(size_t)m * ldq + (size_t)(h0 + r) * dk + d] * scale : 0.f;
	}
	__syncthreads();
	float mx[R], l[R], acc[R][NP][8];
#pragma unroll
	for (int r = 0; r < R; ++r) {
		mx[r] = -INFINITY, l[r] = 0.f;
#pragma unroll
		for (int p = 0; p < NP; ++p)
#pragma unroll
			for (int j = 0; j < 8; ++j) acc[r][p][j] = 0.f;
	}
	const int per = (ntok + nsplit - 1) / nsplit, k_end = min(ntok, (z + 1) * per);
	for (int k0 = z * per + warp * kLaBatch; k0 < k_end; k0 += kLaWarps * kLaBatch) {
		uint4 w[kLaBatch][NP];
#pragma unroll
		for (int b = 0; b < kLaBatch; ++b) {
			const __nv_bfloat16 *row = rows + (size_t)((lo + min(k0 + b, k_end - 1)) % ring) * ld; // past the end: a repeated row with no weight
#pragma unroll
			for (int p = 0; p < NP; ++p) {
				const int c = (lane + 32 * p) * 8;
				w[b][p] = c < dk ? __ldg(reinterpret_cast<const uint4 *>(row + c)) : make_uint4(0, 0, 0, 0);
			}
		}
		float d[kLaBatch][R];
#pragma unroll
		for (int b = 0; b < kLaBatch; ++b) {
#pragma unroll
			for (int r = 0; r < R; ++r) d[b][r] = 0.f;
#pragma unroll
			for (int p = 0; p < NP; ++p) {
				float f[8];
				Elem<YALM_BF16>::unpack(w[b][p], f);
#pragma unroll
				for (int r = 0; r < R; ++r) {
					const float4 q0 = *reinterpret_cast<const float4 *>(qs + r * dkp + (lane + 32 * p) * 8), q1 = *reinterpret_cast<const float4 *>(qs + r * dkp + (lane + 32 * p) * 8 + 4);
					d[b][r] = fmaf(f[0], q0.x, d[b][r]), d[b][r] = fmaf(f[1], q0.y, d[b][r]), d[b][r] = fmaf(f[2], q0.z, d[b][r]), d[b][r] = fmaf(f[3], q0.w, d[b][r]);
					d[b][r] = fmaf(f[4], q1.x, d[b][r]), d[b][r] = fmaf(f[5], q1.y, d[b][r]), d[b][r] = fmaf(f[6], q1.z, d[b][r]), d[b][r] = fmaf(f[7], q1.w, d[b][r]);
				}
			}
		}
#pragma unroll
		for (int o = 16; o > 0; o >>= 1)
#pragma unroll
			for (int b = 0; b < kLaBatch; ++b)
#pragma unroll
				for (int r = 0; r < R; ++r) d[b][r] += __shfl_xor_sync(kFull, d[b][r], o);
		float pw[kLaBatch][R];
#pragma unroll
		for (int r = 0; r < R; ++r) {
			float nm = mx[r];
#pragma unroll
			for (int b = 0; b < kLaBatch; ++b)
				if (k0 + b < k_end) nm = fmaxf(nm, d[b][r]);
			const float corr = mx[r] == -INFINITY ? 0.f : expf(mx[r] - nm);
			float ps = 0.f;
#pragma unroll
			for (int b = 0; b < kLaBatch; ++b) pw[b][r] = k0 + b < k_end ? expf(d[b][r] - nm) : 0.f, ps += pw[b][r];
			l[r] = l[r] * corr + ps, mx[r] = nm;
#pragma unroll
			for (int p = 0; p < NP; ++p)
#pragma unroll
				for (int j = 0; j < 8; ++j) acc[r][p][j] *= corr;
		}
#pragma unroll
		for (int b = 0; b < kLaBatch; ++b)
#pragma unroll
			for (int p = 0; p < NP; ++p) {
				float f[8];
				Elem<YALM_BF16>::unpack(w[b][p], f);
#pragma unroll
				for (int r = 0; r < R; ++r)
#pragma unroll
					for (int j = 0; j < 8; ++j) acc[r][p][j] = fmaf(pw[b][r], f[j], acc[r][p][j]);
			}
	}
#pragma unroll
	for (int r = 0; r < R; ++r) {
#pragma unroll
		for (int p = 0; p < NP; ++p)
#pragma unroll
			for (int j = 0; j < 8; ++j) {
				const int c = (lane + 32 * p) * 8 + j;
				if (c < dv) macc[(warp * R + r) * dv + c] = acc[r][p][j];
			}
		if (lane == 0) mml[(warp * R + r) * 2] = mx[r], mml[(warp * R + r) * 2 + 1] = l[r];
	}
	__syncthreads();
	for (int r = warp; r < nh; r += kLaWarps) { // one warp finishes one head
		float M = -INFINITY;
		for (int w2 = 0; w2 < kLaWarps; ++w2) M = fmaxf(M, mml[(w2 * R + r) * 2]);
		float wt[kLaWarps], L = 0.f;
		for (int w2 = 0; w2 < kLaWarps; ++w2) {
			const float mw = mml[(w2 * R + r) * 2];
			wt[w2] = mw == -INFINITY ? 0.f : expf(mw - M);
			L += wt[w2] * mml[(w2 * R + r) * 2 + 1];
		}
		const int h = h0 + r;
		float *pr = part ? part + ((size_t)(m * n_heads + h) * nsplit + z) * (dv + 2) : nullptr;
		for (int c = lane; c < dv; c += 32) {
			float o = 0.f;
			for (int w2 = 0; w2 < kLaWarps; ++w2) o += wt[w2] * macc[(w2 * R + r) * dv + c];
			if (pr) pr[c] = o;
			else out[(size_t)m * ldo + (size_t)h * dv + c] = o * softmax_finish(M, L, sink, h);
		}
		if (pr && lane == 0) pr[dv] = M, pr[dv + 1] = L;
	}
}
// out[m, h, :] = sum_z w_z acc_z / sum_z w_z L_z with w_z = exp(M_z - max M), splits taken in order (a split without keys has
// M = -inf and no weight).  grid (heads, rows).
__global__ void attn_latent_merge_kernel(float *__restrict__ out, int ldo, const float *__restrict__ part, int n_heads, int dv, int nsplit,
                                         const float *__restrict__ sink) {
	__shared__ float wz[128]; // the splits' weights over the common sum (nsplit <= 128)
	const int h = blockIdx.x, m = blockIdx.y;
	const float *pr = part + (size_t)(m * n_heads + h) * nsplit * (dv + 2);
	if (threadIdx.x < 32) { // lane = split (and split + 32, + 64, + 96)
		const int lane = threadIdx.x;
		float mz[4], lz[4];
#pragma unroll
		for (int k = 0; k < 4; ++k) {
			const int z = lane + 32 * k;
			mz[k] = z < nsplit ? pr[(size_t)z * (dv + 2) + dv] : -INFINITY;
			lz[k] = z < nsplit ? pr[(size_t)z * (dv + 2) + dv + 1] : 0.f;
		}
		const float M = warp_max(fmaxf(fmaxf(mz[0], mz[1]), fmaxf(mz[2], mz[3])));
		float e[4], t[4];
#pragma unroll
		for (int k = 0; k < 4; ++k) e[k] = mz[k] == -INFINITY ? 0.f : expf(mz[k] - M), t[k] = e[k] * lz[k];
		// the sum runs over the splits in order
		float L = 0.f;
		for (int z = 0; z < nsplit; ++z) L += __shfl_sync(kFull, z < 32 ? t[0] : z < 64 ? t[1] : z < 96 ? t[2] : t[3], z & 31);
		const float fin = softmax_finish(M, L, sink, h);
#pragma unroll
		for (int k = 0; k < 4; ++k)
			if (lane + 32 * k < nsplit) wz[lane + 32 * k] = e[k] * fin;
	}
	__syncthreads();
	// grid.z cuts the channels: a thread's loads over the splits are independent, and more CTAs keep more of them in flight
	for (int c = blockIdx.z * blockDim.x + threadIdx.x; c < dv; c += gridDim.z * blockDim.x) {
		float o = 0.f;
#pragma unroll 16
		for (int z = 0; z < nsplit; ++z) o = fmaf(wz[z], pr[(size_t)z * (dv + 2) + c], o);
		out[(size_t)m * ldo + (size_t)h * dv + c] = o;
	}
}

// out[r] = layer norm (or RMS norm) of x[rows[r]] times w   (rows null: r itself)
__global__ void __launch_bounds__(256) layer_norm_gather_rows_kernel(float *__restrict__ out, const float *__restrict__ x, const int *__restrict__ rows,
                                                                     const float *__restrict__ w, int layer_norm, float eps, int dim) {
	__shared__ float red[33];
	const int r = blockIdx.x, m = rows ? rows[r] : r;
	const float *src = x + (size_t)m * dim;
	float mean = 0.f;
	if (layer_norm) {
		float s = 0.f;
		for (int e = threadIdx.x; e < dim; e += blockDim.x) s += src[e];
		mean = block_sum(s, red) / dim;
	}
	float ss = 0.f;
	for (int e = threadIdx.x; e < dim; e += blockDim.x) {
		const float d = src[e] - mean;
		ss += d * d;
	}
	ss = block_sum(ss, red);
	const float sc = 1.0f / sqrtf(ss / dim + eps);
	for (int e = threadIdx.x; e < dim; e += blockDim.x) out[(size_t)r * dim + e] = (src[e] - mean) * sc * w[e];
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

extern "C" int yalm_norm_conv_rows(float *u, float *h, const float *x, const float *w, int layer_norm, float eps, const float *conv_w, float *state, int n,
                                   int dim, int taps, int pos0, const int *ctl, yalm_stream_t s) {
	return yalm_add_norm_conv_rows(u, h, const_cast<float *>(x), nullptr, w, layer_norm, eps, conv_w, state, n, dim, taps, pos0, ctl, s);
}

// The same after x += add (add optional; one launch for one-row calls, a launch of its own before the norm otherwise: a row's
// CTA also reads the rows before it).
extern "C" int yalm_add_norm_conv_rows(float *u, float *h, float *x, const float *add, const float *w, int layer_norm, float eps, const float *conv_w,
                                       float *state, int n, int dim, int taps, int pos0, const int *ctl, yalm_stream_t s) {
	if (add && n > 1) {
		if (int rc = yalm_residual_sum_rows(x, add, nullptr, nullptr, 0, 0, n, dim, s)) return rc;
		add = nullptr;
	}
	if (!u || !h || !x || !w || !conv_w || n < 1 || dim < 1 || taps < 1 || (taps > 1 && !state) || u == x || h == x) return YALM_EINVAL;
	cudaStream_t st = (cudaStream_t)s;
	if (n == 1 && taps <= kOneTaps && dim <= 4 * kOneThreads) {
		if (dim <= kOneThreads) norm_conv_one_kernel<1><<<1, kOneThreads, 0, st>>>(u, h, x, add, w, layer_norm, eps, conv_w, state, dim, taps, pos0, ctl);
		else if (dim <= 2 * kOneThreads) norm_conv_one_kernel<2><<<1, kOneThreads, 0, st>>>(u, h, x, add, w, layer_norm, eps, conv_w, state, dim, taps, pos0, ctl);
		else norm_conv_one_kernel<4><<<1, kOneThreads, 0, st>>>(u, h, x, add, w, layer_norm, eps, conv_w, state, dim, taps, pos0, ctl);
		return (int)cudaGetLastError();
	}
	const size_t smem = sizeof(float) * (size_t)taps * dim;
	if (smem > 160 * 1024) return YALM_EINVAL;
	if (smem > 48 * 1024) YALM_TRY(cudaFuncSetAttribute(norm_conv_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
	norm_conv_rows_kernel<<<n, 256, smem, st>>>(u, h, x, w, layer_norm, eps, conv_w, state, dim, taps, n == 1, pos0, ctl, x, add);
	if (n > 1 && taps > 1) norm_conv_state_kernel<<<(dim + 255) / 256, 256, 0, st>>>(state, h, n, dim, taps, pos0, ctl);
	return (int)cudaGetLastError();
}

extern "C" int yalm_latent_post_rows(float *proj, int ld, int o_q, int q_rank, const float *q_norm, int o_kv, int kv_rank, int rot_dim, const float *kv_norm,
                                     void *ring_buf, int ring, const float *freq, float magnitude, int rot_dims, int interleaved, float eps, int cache_f32,
                                     int n, int pos0, const int *ctl, yalm_stream_t s) {
	if (!proj || n < 1 || q_rank < 0 || (q_rank > 0 && !q_norm) || rot_dims < 0 || rot_dims % 2 || rot_dims > rot_dim || (rot_dims > 0 && !freq) ||
	    (ring_buf && (!kv_norm || kv_rank < 1 || ring < 1)))
		return YALM_EINVAL;
	cudaStream_t st = (cudaStream_t)s;
	if (cache_f32)
		latent_post_rows_kernel<float><<<n, 256, 0, st>>>(proj, ld, o_q, q_rank, q_norm, o_kv, kv_rank, rot_dim, kv_norm, (float *)ring_buf, ring, freq, magnitude,
		                                                  rot_dims, interleaved, eps, pos0, ctl);
	else
		latent_post_rows_kernel<__nv_bfloat16><<<n, 256, 0, st>>>(proj, ld, o_q, q_rank, q_norm, o_kv, kv_rank, rot_dim, kv_norm, (__nv_bfloat16 *)ring_buf, ring,
		                                                          freq, magnitude, rot_dims, interleaved, eps, pos0, ctl);
	return (int)cudaGetLastError();
}

extern "C" int yalm_latent_query_rows(float *out, int ldo, const float *q, int ldq, const void *uk, int dtype, int n, int heads, int dim, int rot_dim,
                                      int kv_rank, const float *freq, float magnitude, int rot_dims, int interleaved, int pos0, const int *ctl,
                                      yalm_stream_t s) {
	if (!out || !q || (!uk && dim > 0) || n < 1 || heads < 1 || dim < 0 || rot_dim < 0 || kv_rank < 1 || rot_dims < 0 || rot_dims % 2 || rot_dims > rot_dim ||
	    (rot_dims > 0 && !freq))
		return YALM_EINVAL;
	const size_t smem = sizeof(float) * kLqRows * (size_t)(dim + rot_dim);
	if (smem > 48 * 1024) return YALM_EINVAL;
	const dim3 grid(heads, (n + kLqRows - 1) / kLqRows, (kv_rank + 63) / 64);
	DISPATCH_DT(dtype, (latent_query_rows_kernel<DT><<<grid, 64, smem, (cudaStream_t)s>>>(out, ldo, q, ldq, uk, n, dim, rot_dim, kv_rank, freq, magnitude,
	                                                                                      rot_dims, interleaved, pos0, ctl)));
	return (int)cudaGetLastError();
}

extern "C" int yalm_head_linear_gate_rows(float *out, int ldo, const float *x, int ldx, const void *w, int dtype, const float *gate, int ldg, int n, int heads,
                                          int N, int K, yalm_stream_t s) {
	if (!out || !x || !w || n < 1 || heads < 1 || N < 1 || K < 1) return YALM_EINVAL;
	const size_t smem = sizeof(float) * kHlRows * (size_t)K;
	if (smem > 48 * 1024) return YALM_EINVAL;
	const int rb = (n + kHlRows - 1) / kHlRows;
	const dim3 grid(heads, rb, heads * rb >= 296 ? 1 : std::min((N + 7) / 8, (296 + heads * rb - 1) / (heads * rb))); // few rows: the outputs spread over more CTAs
	DISPATCH_DT(dtype, (head_linear_gate_rows_kernel<DT><<<grid, 256, smem, (cudaStream_t)s>>>(out, ldo, x, ldx, w, gate, ldg, n, N, K)));
	return (int)cudaGetLastError();
}

extern "C" int yalm_gla_prep_rows(float *z, int ldz, const float *bias, float tau, float *q, int ldq, float q_scale, int n, int channels, yalm_stream_t s) {
	if (!z || !bias || !q || !(tau > 0.f) || n < 1 || channels < 1) return YALM_EINVAL;
	gla_prep_rows_kernel<<<dim3((channels + 255) / 256, n), 256, 0, (cudaStream_t)s>>>(z, ldz, bias, 1.0f / tau, q, ldq, q_scale, channels);
	return (int)cudaGetLastError();
}

extern "C" int yalm_depth_average_rows(float *x, float *hist, size_t stride, const float *w, int count, int n, int dim, const float *a, const float *b,
                                       const float *y, int ldy, int nsum, yalm_stream_t s) {
	if (!x || !hist || count < 1 || n < 1 || dim < 1 || stride < (size_t)n * dim || (y && nsum < 1)) return YALM_EINVAL;
	const size_t total = (size_t)n * dim;
	depth_average_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)s>>>(x, hist, stride, w, count, total, a, b, y, ldy, nsum, dim);
	return (int)cudaGetLastError();
}

extern "C" int yalm_layer_norm_gather_rows(float *out, const float *x, const int *rows, const float *w, int layer_norm, float eps, int n_rows, int dim,
                                           yalm_stream_t s) {
	if (!out || !x || !w || n_rows < 1 || dim < 1) return YALM_EINVAL;
	layer_norm_gather_rows_kernel<<<n_rows, 256, 0, (cudaStream_t)s>>>(out, x, rows, w, layer_norm, eps, dim);
	return (int)cudaGetLastError();
}

extern "C" int yalm_latent_gather_rows16(void *out16, const void *ring_buf, int ring, int row, int kv_rank, int first_pos, int count, yalm_stream_t s) {
	if (!out16 || !ring_buf || ring < 1 || kv_rank < 1 || row < kv_rank || first_pos < 0 || count < 1 || count > ring) return YALM_EINVAL;
	latent_gather_rows_kernel<<<count, 128, 0, (cudaStream_t)s>>>((__nv_bfloat16 *)out16, (const __nv_bfloat16 *)ring_buf, ring, row, kv_rank, first_pos);
	return (int)cudaGetLastError();
}

extern "C" int yalm_latent_pack_rings(void *key_ring, void *value_ring, const float *kv, int ldkv, const void *ring_buf, int ring, int kv_rank, int rot_dim,
                                      int heads, int dim, int vdim, int ring_out, int first_pos, int count, yalm_stream_t s) {
	if (!key_ring || !value_ring || !kv || !ring_buf || ring < 1 || ring_out < 1 || heads < 1 || dim < 0 || vdim < 1 || first_pos < 0 || count < 1 ||
	    count > ring || count > ring_out)
		return YALM_EINVAL;
	latent_pack_rings_kernel<<<count, 256, 0, (cudaStream_t)s>>>((__nv_bfloat16 *)key_ring, (__nv_bfloat16 *)value_ring, kv, ldkv,
	                                                             (const __nv_bfloat16 *)ring_buf, ring, kv_rank + rot_dim, kv_rank, rot_dim, heads, dim, vdim,
	                                                             ring_out, first_pos);
	return (int)cudaGetLastError();
}

extern "C" int yalm_rotate_heads_rows(float *q, int ldq, int heads, int head_size, int offset, const float *freq, float magnitude, int rot_dims,
                                      int interleaved, int n, int pos0, const int *ctl, yalm_stream_t s) {
	if (!q || n < 1 || heads < 1 || rot_dims < 0 || rot_dims % 2 || offset < 0 || offset + rot_dims > head_size || (rot_dims > 0 && !freq)) return YALM_EINVAL;
	if (rot_dims == 0) return 0;
	rotate_heads_rows_kernel<<<n, 128, 0, (cudaStream_t)s>>>(q, ldq, heads, head_size, offset, freq, magnitude, rot_dims, interleaved, pos0, ctl);
	return (int)cudaGetLastError();
}

extern "C" int yalm_sigmoid_gate_rows(float *x, int ldx, const float *gate, int ldg, int n, int dim, yalm_stream_t s) {
	if (!x || !gate || n < 1 || dim < 1) return YALM_EINVAL;
	sigmoid_gate_rows_kernel<<<dim3((dim + 255) / 256, n), 256, 0, (cudaStream_t)s>>>(x, ldx, gate, ldg, dim);
	return (int)cudaGetLastError();
}

// 1 when yalm_attn_latent_rows has a kernel for these sizes (bf16 rows of 16-byte pieces, at most 768 channels).
extern "C" int yalm_attn_latent_rows_shape(int dk, int dv, int ld) {
	return dk >= 8 && dk <= 768 && dk % 8 == 0 && dv >= 1 && dv <= dk && ld >= dk && ld % 8 == 0;
}

template <int R, int NP>
static int launch_attn_latent(float *out, int ldo, const float *q, int ldq, const void *rows, int ld, float *ws, int n, int n_heads, int dk, int dv, int ring,
                              int window, float scale, int nsplit, int pos0, const int *ctl, const float *sink, cudaStream_t st) {
	const size_t smem = sizeof(float) * ((size_t)R * NP * 256 + (size_t)kLaWarps * R * dv + kLaWarps * R * 2);
	if (smem > 96 * 1024) return YALM_EINVAL;
	if (smem > 48 * 1024) YALM_TRY(cudaFuncSetAttribute(attn_latent_rows_kernel<R, NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
	attn_latent_rows_kernel<R, NP><<<dim3((n_heads + R - 1) / R, n, nsplit), kLaWarps * 32, smem, st>>>(out, ldo, q, ldq, (const __nv_bfloat16 *)rows, ld,
	                                                                                                  nsplit > 1 ? ws : nullptr, n_heads, dk, dv, ring,
	                                                                                                  window, scale, pos0, ctl, sink);
	if (nsplit > 1) attn_latent_merge_kernel<<<dim3(n_heads, n, (dv + 127) / 128), 128, 0, st>>>(out, ldo, ws, n_heads, dv, nsplit, sink);
	return (int)cudaGetLastError();
}

// Attention of n query rows (n_heads x dk each) over cached bf16 rows shared by all heads: key = the row's dk channels, value =
// its first dv; position i sees rows j with 0 <= i - j < window (0: all).  workspace: yalm_attn_window_pool_workspace(dv) floats
// (split partials of calls with few rows), or null.
extern "C" int yalm_attn_latent_rows(float *out, int ldo, const float *q, int ldq, const void *rows, int ld, float *workspace, int n, int n_heads, int dk,
                                     int dv, int ring, int window, float scale, int context, int pos0, const int *ctl, yalm_stream_t s) {
	return yalm_attn_latent_rows_sink(out, ldo, q, ldq, rows, ld, workspace, n, n_heads, dk, dv, ring, window, scale, context, pos0, ctl, nullptr, s);
}

// The same with a sink per head in the softmax's denominator (null: none).
extern "C" int yalm_attn_latent_rows_sink(float *out, int ldo, const float *q, int ldq, const void *rows, int ld, float *workspace, int n, int n_heads, int dk,
                                          int dv, int ring, int window, float scale, int context, int pos0, const int *ctl, const float *sink, yalm_stream_t s) {
	if (!out || !q || !rows || n < 1 || n_heads < 1 || ring < 1 || !yalm_attn_latent_rows_shape(dk, dv, ld) || ((uintptr_t)rows & 15)) return YALM_EINVAL;
	const int R = n_heads >= 4 ? 4 : n_heads >= 2 ? 2 : 1, hg = (n_heads + R - 1) / R, NP = (dk / 8 + 31) / 32;
	int nsplit = 1;
	const int ctas = hg * n;
	if (workspace && ctas < 296) { // few rows: split the keys so that every SM has work; the count depends on shapes only
		const int most = window > 0 ? window : (context > 0 ? context : ring);
		const int batches = (most + kLaWarps * kLaBatch - 1) / (kLaWarps * kLaBatch);
		nsplit = std::max(1, std::min({(296 + ctas - 1) / ctas, batches, kLaMaxParts / (n * n_heads), 32}));
	}
	cudaStream_t st = (cudaStream_t)s;
#define LA_CASE(R_, NP_)                                                                                                              \
	if (R == R_ && NP == NP_) return launch_attn_latent<R_, NP_>(out, ldo, q, ldq, rows, ld, workspace, n, n_heads, dk, dv, ring, window, scale, nsplit, pos0, ctl, sink, st)
	LA_CASE(4, 1); LA_CASE(4, 2); LA_CASE(4, 3); LA_CASE(2, 1); LA_CASE(2, 2); LA_CASE(2, 3); LA_CASE(1, 1); LA_CASE(1, 2); LA_CASE(1, 3);
#undef LA_CASE
	return YALM_EINVAL;
}

// Joins nsplit (<= 128) partials per (row, head) of (dv accumulators, max, sum) in `part`, in order, sink included (null: none).
extern "C" int yalm_attn_latent_merge(float *out, int ldo, const float *part, int n, int n_heads, int dv, int nsplit, const float *sink, yalm_stream_t s) {
	if (!out || !part || n < 1 || n_heads < 1 || dv < 1 || nsplit < 1 || nsplit > 128) return YALM_EINVAL;
	attn_latent_merge_kernel<<<dim3(n_heads, n, (dv + 127) / 128), 128, 0, (cudaStream_t)s>>>(out, ldo, part, n_heads, dv, nsplit, sink);
	return (int)cudaGetLastError();
}
