// Row kernels of the layered executor for layers with a norm before and after every sublayer (stack.cpp:
// stack_layer_sandwich): attention heads with a per-head q / k norm and rotary positions appended to key / value rings and to
// the buffers of a window's kept first tokens; the combination of two softmax maps into one differential head output; a plain
// (not gated) activation; and the per-layer token side input.  Every op takes n rows = n consecutive positions of one sequence.
// Norms, angles, rotation, the maps' difference and the residual stream are fp32.
#include "stack_rows.cuh"

#include <cuda_bf16.h>

namespace yalm {
namespace stack {

// ---- per-head q / k norm, rotary positions, cache append ----------------------------------------------------------------------
// Row m of the packed projection P (ld): nqv query vectors of dk channels from o_q, nkv key vectors from o_k, nvh value heads
// of dv channels from o_v.  Every query and key vector: RMS norm over its dk channels with the shared weight qw / kw (null:
// none), then its first rot_dims channels turned by the row's position (pair i = channels (i, i + rot_dims / 2), or
// (2 i, 2 i + 1) if interleaved).  Queries stay in place; key vector j goes to kring (j, slot, channel), value head j to vring;
// positions below `keep` also go, as the ring holds them, to kfirst (j, keep, dk) / vfirst (j, keep, dv) in fp32, from where
// the attention reads the tokens that stay visible after they have left the window.  A warp owns a vector.
constexpr int kHnWarps = 8, kHnMaxDim = 512;
template <typename CT>
__global__ void __launch_bounds__(kHnWarps * 32) head_norm_rope_append_rows_kernel(float *__restrict__ P, int ld, int o_q, int o_k, int o_v, int nqv, int nkv,
                                                                                  int nvh, int dk, int dv, const float *__restrict__ qw,
                                                                                  const float *__restrict__ kw, const float *__restrict__ freq, float mag,
                                                                                  int rot_dims, int interleaved, float eps, CT *__restrict__ kring,
                                                                                  CT *__restrict__ vring, int ring, float *__restrict__ kfirst,
                                                                                  float *__restrict__ vfirst, int keep, int pos0,
                                                                                  const int *__restrict__ ctl) {
	__shared__ float buf[kHnWarps][kHnMaxDim];
	const int m = blockIdx.x, p = first_pos(ctl, pos0) + m, slot = p % ring;
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, half = rot_dims / 2;
	float *row = P + (size_t)m * ld, *vs = buf[warp];
	for (int v = blockIdx.y * kHnWarps + warp; v < nqv + nkv; v += gridDim.y * kHnWarps) { // grid.y spreads a row's vectors over CTAs
		const bool is_q = v < nqv;
		float *src = row + (is_q ? o_q + (size_t)v * dk : o_k + (size_t)(v - nqv) * dk);
		const float *w = is_q ? qw : kw;
		float ss = 0.f;
		for (int d = lane; d < dk; d += 32) {
			const float x = src[d];
			vs[d] = x, ss += x * x;
		}
		ss = warp_sum(ss);
		const float r = w ? 1.0f / sqrtf(ss / (float)dk + eps) : 1.f;
		if (w)
			for (int d = lane; d < dk; d += 32) vs[d] = vs[d] * r * w[d];
		__syncwarp();
		CT *kdst = is_q ? nullptr : kring + ((size_t)(v - nqv) * ring + slot) * dk;
		float *fdst = (!is_q && p < keep) ? kfirst + ((size_t)(v - nqv) * keep + p) * dk : nullptr;
		for (int d = lane; d < dk; d += 32) {
			float o = vs[d];
			if (d < rot_dims) {
				const int i = interleaved ? d >> 1 : (d < half ? d : d - half);
				const bool first = interleaved ? !(d & 1) : d < half;
				const float a = vs[interleaved ? 2 * i : i], b = vs[interleaved ? 2 * i + 1 : i + half];
				float sn, cs;
				sincosf((float)p * freq[i], &sn, &cs);
				sn *= mag, cs *= mag;
				o = first ? a * cs - b * sn : b * cs + a * sn;
			}
			if (is_q) src[d] = o;
			else {
				cache_put(kdst, d, o);
				if (fdst) fdst[d] = cache_get(kdst, d);
			}
		}
		__syncwarp();
	}
	for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < nvh * dv; e += gridDim.y * blockDim.x) {
		const int g = e / dv, d = e % dv;
		CT *dst = vring + ((size_t)g * ring + slot) * dv;
		cache_put(dst, d, row[o_v + e]);
		if (p < keep) vfirst[((size_t)g * keep + p) * dv + d] = cache_get(dst, d);
	}
}

// ---- two softmax maps into one head output ------------------------------------------------------------------------------------
// a (n, 2 heads dv): the first map's outputs of all heads, then the second map's.  Per head o = a_1 - lambda a_2,
// out = o / sqrt(mean o^2 + eps) * out_scale * sigmoid(gate[m, h]) (gate null: none).  A warp owns a head.
__global__ void __launch_bounds__(256) diff_combine_rows_kernel(float *__restrict__ out, int ldo, const float *__restrict__ a, int lda,
                                                                const float *__restrict__ gate, int ldg, int heads, int dv, float lambda, float out_scale,
                                                                float eps) {
	const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	for (int h = warp; h < heads; h += blockDim.x >> 5) {
		const float *a1 = a + (size_t)m * lda + (size_t)h * dv, *a2 = a1 + (size_t)heads * dv;
		float ss = 0.f;
		for (int c = lane; c < dv; c += 32) {
			const float o = a1[c] - lambda * a2[c];
			ss += o * o;
		}
		ss = warp_sum(ss);
		float f = out_scale / sqrtf(ss / (float)dv + eps);
		if (gate) f *= 1.0f / (1.0f + expf(-gate[(size_t)m * ldg + h]));
		for (int c = lane; c < dv; c += 32) out[(size_t)m * ldo + (size_t)h * dv + c] = (a1[c] - lambda * a2[c]) * f;
	}
}

// ---- a plain activation, in place ---------------------------------------------------------------------------------------------
__global__ void act_rows_kernel(float *__restrict__ h, int ld, int ff, int act) {
	float *row = h + (size_t)blockIdx.y * ld;
	for (int f = blockIdx.x * blockDim.x + threadIdx.x; f < ff; f += gridDim.x * blockDim.x) row[f] = act_value(row[f], act);
}

// ---- token side input -------------------------------------------------------------------------------------------------------
// x[m] += rms(y) * nw with y = P (gelu_tanh(G x[m]) * e), e = table[token, col0 .. col0 + sd): G (sd, dim), P (dim, sd), the
// table (vocab, ldt) in the weight type.  One CTA per row: warps take the sd gate rows, threads the dim outputs.
template <int DT>
__global__ void __launch_bounds__(256) token_side_rows_kernel(float *__restrict__ x, const void *__restrict__ table, int ldt, int col0,
                                                              const int *__restrict__ tokens, const int *__restrict__ ctl, const void *__restrict__ wg,
                                                              const void *__restrict__ wp, const float *__restrict__ nw, int dim, int sd, float eps) {
	extern __shared__ __align__(16) float sms[];
	__shared__ float red[33];
	float *xs = sms, *g = xs + ((dim + 3) & ~3), *ys = g + ((sd + 3) & ~3);
	const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int token = tokens ? tokens[m] : ctl[CTL_TOKEN];
	float *row = x + (size_t)m * dim;
	for (int e = threadIdx.x; e < dim; e += blockDim.x) xs[e] = row[e];
	__syncthreads();
	const bool vec = dim % Elem<DT>::VEC == 0 && aligned16(wg) && ((size_t)dim * sizeof(typename Elem<DT>::T)) % 16 == 0;
	for (int j = warp; j < sd; j += blockDim.x >> 5) {
		const float z = warp_dot<DT>(wg, (size_t)j * dim, xs, dim, vec);
		if (lane == 0) g[j] = act_value(z, 3) * Elem<DT>::get(table, (size_t)token * ldt + col0 + j);
	}
	__syncthreads();
	float ss = 0.f;
	for (int e = threadIdx.x; e < dim; e += blockDim.x) {
		float y = 0.f;
		for (int j = 0; j < sd; ++j) y = fmaf(Elem<DT>::get(wp, (size_t)e * sd + j), g[j], y);
		ys[e] = y, ss += y * y;
	}
	ss = block_sum(ss, red);
	const float r = 1.0f / sqrtf(ss / (float)dim + eps);
	for (int e = threadIdx.x; e < dim; e += blockDim.x) row[e] += ys[e] * r * nw[e];
}


// The same in two steps that spread over the GPU, for sizes that are 16-byte multiples: h = gelu_tanh(G x) * e (a warp per gate
// row and row of x; or, after a tensor-core product g = x G^T, in place), then the products' usual routes for y = P h and the norm.
template <int DT>
__global__ void __launch_bounds__(128) token_side_gate_rows_kernel(float *__restrict__ h, int ldh, const float *__restrict__ x, int ldx,
                                                                   const void *__restrict__ table, int ldt, int col0, const int *__restrict__ tokens,
                                                                   const int *__restrict__ ctl, const void *__restrict__ wg, int dim, int sd) {
	const int m = blockIdx.y, j = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
	if (j >= sd) return;
	const float z = warp_dot<DT>(wg, (size_t)j * dim, x + (size_t)m * ldx, dim, true);
	if ((threadIdx.x & 31) == 0) {
		const int token = tokens ? tokens[m] : ctl[CTL_TOKEN];
		h[(size_t)m * ldh + j] = act_value(z, 3) * Elem<DT>::get(table, (size_t)token * ldt + col0 + j);
	}
}
template <int DT>
__global__ void token_side_act_rows_kernel(float *__restrict__ h, int ldh, const void *__restrict__ table, int ldt, int col0, const int *__restrict__ tokens,
                                           const int *__restrict__ ctl, int sd) {
	const int m = blockIdx.y;
	const int token = tokens ? tokens[m] : ctl[CTL_TOKEN];
	for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < sd; j += gridDim.x * blockDim.x)
		h[(size_t)m * ldh + j] = act_value(h[(size_t)m * ldh + j], 3) * Elem<DT>::get(table, (size_t)token * ldt + col0 + j);
}

} // namespace stack
} // namespace yalm

using namespace yalm;
using namespace yalm::stack;

extern "C" int yalm_head_norm_rope_append_rows(float *proj, int ld, int o_q, int o_k, int o_v, int n_q_vectors, int n_k_vectors, int n_v_heads, int dk, int dv,
                                               const float *q_norm, const float *k_norm, const float *freq, float magnitude, int rot_dims, int interleaved,
                                               float eps, void *key_ring, void *value_ring, int ring, float *key_first, float *value_first, int keep,
                                               int cache_f32, int n, int pos0, const int *ctl, yalm_stream_t s) {
	if (!proj || !key_ring || !value_ring || n < 1 || ring < 1 || dk < 1 || dk > kHnMaxDim || dv < 1 || rot_dims < 0 || rot_dims > dk || rot_dims % 2 ||
	    (rot_dims > 0 && !freq) || keep < 0 || (keep > 0 && (!key_first || !value_first)))
		return YALM_EINVAL;
	cudaStream_t st = (cudaStream_t)s;
	// every load of a vector's chain (channels, norm, rotation, store) waits for the one before it: enough warps in flight hide that
	const dim3 grid(n, std::max(1, std::min((n_q_vectors + n_k_vectors + kHnWarps - 1) / kHnWarps, n >= 64 ? 4 : 16)));
	if (cache_f32)
		head_norm_rope_append_rows_kernel<float><<<grid, kHnWarps * 32, 0, st>>>(proj, ld, o_q, o_k, o_v, n_q_vectors, n_k_vectors, n_v_heads, dk, dv, q_norm, k_norm,
		                                                                       freq, magnitude, rot_dims, interleaved, eps, (float *)key_ring, (float *)value_ring,
		                                                                       ring, key_first, value_first, keep, pos0, ctl);
	else
		head_norm_rope_append_rows_kernel<__nv_bfloat16><<<grid, kHnWarps * 32, 0, st>>>(proj, ld, o_q, o_k, o_v, n_q_vectors, n_k_vectors, n_v_heads, dk, dv, q_norm,
		                                                                               k_norm, freq, magnitude, rot_dims, interleaved, eps,
		                                                                               (__nv_bfloat16 *)key_ring, (__nv_bfloat16 *)value_ring, ring, key_first,
		                                                                               value_first, keep, pos0, ctl);
	return (int)cudaGetLastError();
}

extern "C" int yalm_diff_combine_rows(float *out, int ldo, const float *maps, int ldm, const float *gate, int ldg, int n, int heads, int dv, float lambda,
                                      float out_scale, float eps, yalm_stream_t s) {
	if (!out || !maps || n < 1 || heads < 1 || dv < 1) return YALM_EINVAL;
	diff_combine_rows_kernel<<<n, 256, 0, (cudaStream_t)s>>>(out, ldo, maps, ldm, gate, ldg, heads, dv, lambda, out_scale, eps);
	return (int)cudaGetLastError();
}

extern "C" int yalm_act_rows(float *h, int ld, int n, int ff, int act, yalm_stream_t s) {
	if (!h || n < 1 || ff < 1 || ld < ff) return YALM_EINVAL;
	act_rows_kernel<<<dim3(std::min(64, (ff + 255) / 256), n), 256, 0, (cudaStream_t)s>>>(h, ld, ff, act);
	return (int)cudaGetLastError();
}

extern "C" int yalm_token_side_rows(float *x, const void *table, int ldt, int col0, const int *tokens, const int *ctl, const void *w_gate, const void *w_proj,
                                    const float *norm_w, int dtype, int n, int dim, int side, float eps, yalm_stream_t s) {
	if (!x || !table || (!tokens && !ctl) || !w_gate || !w_proj || !norm_w || n < 1 || dim < 1 || side < 1 || col0 < 0 || col0 + side > ldt) return YALM_EINVAL;
	const size_t smem = sizeof(float) * (2 * (size_t)((dim + 3) & ~3) + ((side + 3) & ~3));
	if (smem > 200 * 1024) return YALM_EINVAL;
	cudaStream_t st = (cudaStream_t)s;
#define SIDE_CASE(DT_)                                                                                                                \
	{                                                                                                                                 \
		if (smem > 48 * 1024) YALM_TRY(cudaFuncSetAttribute(token_side_rows_kernel<DT_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
		token_side_rows_kernel<DT_><<<n, 256, smem, st>>>(x, table, ldt, col0, tokens, ctl, w_gate, w_proj, norm_w, dim, side, eps);  \
	}
	if (dtype == YALM_F32) SIDE_CASE(YALM_F32)
	else if (dtype == YALM_F16) SIDE_CASE(YALM_F16)
	else if (dtype == YALM_BF16) SIDE_CASE(YALM_BF16)
	else return YALM_EINVAL;
#undef SIDE_CASE
	return (int)cudaGetLastError();
}

// h[m, j] = gelu_tanh(w_gate[j] . x[m]) * table[token of row m, col0 + j] (g NULL), or the same from a product g = x w_gate^T that
// h already holds (w_gate NULL).  dim % 8 == 0 (fp32: 4), 16-byte aligned rows.
extern "C" int yalm_token_side_gate_rows(float *h, int ldh, const float *x, int ldx, const void *table, int ldt, int col0, const int *tokens, const int *ctl,
                                         const void *w_gate, int dtype, int n, int dim, int side, yalm_stream_t s) {
	if (!h || !table || (!tokens && !ctl) || n < 1 || side < 1 || col0 < 0 || col0 + side > ldt) return YALM_EINVAL;
	cudaStream_t st = (cudaStream_t)s;
	if (!w_gate) {
		const dim3 grid(std::min(8, (side + 127) / 128), n);
		if (dtype == YALM_F32) token_side_act_rows_kernel<YALM_F32><<<grid, 128, 0, st>>>(h, ldh, table, ldt, col0, tokens, ctl, side);
		else if (dtype == YALM_F16) token_side_act_rows_kernel<YALM_F16><<<grid, 128, 0, st>>>(h, ldh, table, ldt, col0, tokens, ctl, side);
		else if (dtype == YALM_BF16) token_side_act_rows_kernel<YALM_BF16><<<grid, 128, 0, st>>>(h, ldh, table, ldt, col0, tokens, ctl, side);
		else return YALM_EINVAL;
		return (int)cudaGetLastError();
	}
	const int vec = dtype == YALM_F32 ? 4 : 8;
	if (!x || dim < 1 || dim % vec || ldx % 4 || ((uintptr_t)x & 15) || ((uintptr_t)w_gate & 15)) return YALM_EINVAL;
	const dim3 grid((side + 3) / 4, n);
	if (dtype == YALM_F32) token_side_gate_rows_kernel<YALM_F32><<<grid, 128, 0, st>>>(h, ldh, x, ldx, table, ldt, col0, tokens, ctl, w_gate, dim, side);
	else if (dtype == YALM_F16) token_side_gate_rows_kernel<YALM_F16><<<grid, 128, 0, st>>>(h, ldh, x, ldx, table, ldt, col0, tokens, ctl, w_gate, dim, side);
	else if (dtype == YALM_BF16) token_side_gate_rows_kernel<YALM_BF16><<<grid, 128, 0, st>>>(h, ldh, x, ldx, table, ldt, col0, tokens, ctl, w_gate, dim, side);
	else return YALM_EINVAL;
	return (int)cudaGetLastError();
}
