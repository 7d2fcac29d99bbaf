// Device pieces shared by the layered executor's row kernels (ops_stack.cu) and by the one-row GEMV with a fused tail
// (ops_stack_gemv.cu): element access for fp32 / fp16 / bf16 weights and caches, and the per-row bodies of the q / k norm +
// value blending + cache append, of the block means, of the output norm + residual, and of the gated activation.
#pragma once

#include "common.cuh"

#include <cuda_bf16.h>

#include "gemv.cuh"

namespace yalm {
namespace stack {

// ---- element access ----------------------------------------------------------------------------------------------------
template <int DT> struct Elem;
template <> struct Elem<YALM_F32> {
	using T = float;
	static constexpr int VEC = 4;
	__device__ static __forceinline__ float get(const void *p, size_t i) { return static_cast<const float *>(p)[i]; }
	__device__ static __forceinline__ void unpack(uint4 w, float (&f)[8]) {
		f[0] = __uint_as_float(w.x), f[1] = __uint_as_float(w.y), f[2] = __uint_as_float(w.z), f[3] = __uint_as_float(w.w);
	}
};
template <> struct Elem<YALM_F16> {
	using T = __half;
	static constexpr int VEC = 8;
	__device__ static __forceinline__ float get(const void *p, size_t i) { return __half2float(static_cast<const __half *>(p)[i]); }
	__device__ static __forceinline__ void unpack(uint4 w, float (&f)[8]) {
		const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
		for (int i = 0; i < 4; ++i) {
			const float2 v = __half22float2(*reinterpret_cast<const __half2 *>(&u[i]));
			f[2 * i] = v.x, f[2 * i + 1] = v.y;
		}
	}
};
template <> struct Elem<YALM_BF16> {
	using T = __nv_bfloat16;
	static constexpr int VEC = 8;
	__device__ static __forceinline__ float get(const void *p, size_t i) {
		return __uint_as_float((uint32_t) static_cast<const uint16_t *>(p)[i] << 16);
	}
	__device__ static __forceinline__ void unpack(uint4 w, float (&f)[8]) { // bf16 -> fp32 is a 16-bit shift
		const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
		for (int i = 0; i < 4; ++i) f[2 * i] = __uint_as_float(u[i] << 16), f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
	}
};

__device__ __forceinline__ float cache_get(const float *p, size_t i) { return p[i]; }
__device__ __forceinline__ float cache_get(const __nv_bfloat16 *p, size_t i) {
	return __uint_as_float((uint32_t) reinterpret_cast<const uint16_t *>(p)[i] << 16);
}
__device__ __forceinline__ void cache_put(float *p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void cache_put(__nv_bfloat16 *p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ int first_pos(const int *ctl, int pos0) { return ctl ? ctl[CTL_POS] : pos0; }

// A sink joins the softmax's denominator as exp(sink) without a key or a value: the factor on an accumulator whose weights
// are exp(score - M) and sum to L is 1 / (L + exp(sink - M)), formed over the larger of M and the sink so that nothing overflows.
__device__ __forceinline__ float softmax_finish(float M, float L, const float *sink, int h) {
	if (!sink) return 1.0f / L;
	const float sk = sink[h], top = fmaxf(M, sk), f = expf(M - top);
	return f / (L * f + expf(sk - top));
}

__host__ __device__ inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// dot(weight row, x) over K elements, result in every lane.  `vec`: the row and x are 16-byte aligned and K % VEC == 0.
template <int DT>
__device__ __forceinline__ float warp_dot(const void *w, size_t row_off, const float *__restrict__ x, int K, bool vec) {
	using E = Elem<DT>;
	const int lane = threadIdx.x & 31;
	float acc = 0.f;
	if (vec) {
		const typename E::T *row = static_cast<const typename E::T *>(w) + row_off;
		constexpr int U = 4, STEP = 32 * E::VEC; // U loads in flight per lane before the first multiply
		for (int k0 = lane * E::VEC; k0 < K; k0 += U * STEP) {
			uint4 wv[U];
			float4 xv[U][E::VEC / 4]; // the inputs are fetched with the weights: one memory round trip per batch, not one per piece
#pragma unroll
			for (int u = 0; u < U; ++u)
				if (k0 + u * STEP < K) {
					wv[u] = ldg_stream(row + k0 + u * STEP);
#pragma unroll
					for (int i = 0; i < E::VEC / 4; ++i) xv[u][i] = *reinterpret_cast<const float4 *>(x + k0 + u * STEP + 4 * i);
				}
#pragma unroll
			for (int u = 0; u < U; ++u)
				if (k0 + u * STEP < K) {
					float f[8];
					E::unpack(wv[u], f);
#pragma unroll
					for (int i = 0; i < E::VEC / 4; ++i) {
						acc = fmaf(f[4 * i], xv[u][i].x, acc), acc = fmaf(f[4 * i + 1], xv[u][i].y, acc);
						acc = fmaf(f[4 * i + 2], xv[u][i].z, acc), acc = fmaf(f[4 * i + 3], xv[u][i].w, acc);
					}
				}
		}
	} else {
		for (int k = lane; k < K; k += 32) acc = fmaf(E::get(w, row_off + k), x[k], acc);
	}
	return warp_sum(acc);
}


__device__ __forceinline__ float glu_value(float g, float u, int act, float alpha, float limit, float up_offset) {
	if (limit > 0.f) g = fminf(g, limit), u = fminf(fmaxf(u, -limit), limit);
	float a;
	if (act == 2) a = g / (1.0f + expf(-alpha * g));      // g * sigmoid(alpha g)
	else if (act == 3) a = 0.5f * g * (1.0f + tanhf(0.7978845608f * (g + 0.044715f * g * g * g))); // tanh GELU, sqrt(2 / pi) to fp32 precision
	else if (act == YALM_ACT_SILU) a = act_silu(g);
	else a = act_gelu(g);
	return a * (u + up_offset);
}

// a plain activation: 4 the exact GELU, 3 the tanh GELU, else SiLU / the .yalm models' GELU
__device__ __forceinline__ float act_value(float z, int act) {
	if (act == 4) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752f));                                   // exact GELU
	if (act == 3) return 0.5f * z * (1.0f + tanhf(0.7978845608f * (z + 0.044715f * z * z * z)));              // tanh GELU
	if (act == YALM_ACT_SILU) return act_silu(z);
	return act_gelu(z);
}

// Row `row` of q | k | v (fp32) at ring slot `slot`: RMS norm over the WHOLE q and k projections (all heads at once), one
// weight per channel (qnorm / knorm null: left as they are); q stays in place, k goes to the ring.  v: vmode 1 keeps a copy
// in vfirst (the first blending layer), vmode 2 blends v = (1 - lambda) v + lambda vfirst (later blending layers); the
// blended v is what is cached.  Caches are head-major (kv head, slot, channel).  All threads of the CTA take part.  The row
// is read past L1 (__ldcg): in the fused tail other CTAs of the same launch wrote it.
template <typename CT>
__device__ __forceinline__ void qkv_post_row(float *row, CT *kc, CT *vc, float *vfirst, const float *qnorm, const float *knorm, const float *vmix, int vmode,
                                             int nq, int nk, int nv, int dk, int dv, int ring, int slot, float eps, float *red) {
	float rq = 1.f, rk = 1.f;
	if (qnorm) {
		float s = 0.f;
		for (int e = threadIdx.x; e < nq; e += blockDim.x) s += __ldcg(row + e) * __ldcg(row + e);
		s = block_sum(s, red);
		rq = 1.0f / sqrtf(s / nq + eps);
	}
	if (knorm) {
		float s = 0.f;
		for (int e = threadIdx.x; e < nk; e += blockDim.x) s += __ldcg(row + nq + e) * __ldcg(row + nq + e);
		s = block_sum(s, red);
		rk = 1.0f / sqrtf(s / nk + eps);
	}
	if (qnorm)
		for (int e = threadIdx.x; e < nq; e += blockDim.x) row[e] = __ldcg(row + e) * rq * qnorm[e];
	for (int e = threadIdx.x; e < nk; e += blockDim.x) {
		float v = __ldcg(row + nq + e);
		if (knorm) v = v * rk * knorm[e];
		const int g = e / dk, d = e % dk;
		cache_put(kc, ((size_t)g * ring + slot) * dk + d, v);
	}
	const float lam = vmode == 2 ? vmix[0] : 0.f;
	for (int e = threadIdx.x; e < nv; e += blockDim.x) {
		float v = __ldcg(row + nq + nk + e);
		if (vmode == 1) vfirst[e] = v;
		else if (vmode == 2) v = (1.0f - lam) * v + lam * vfirst[e];
		const int g = e / dv, d = e % dv;
		cache_put(vc, ((size_t)g * ring + slot) * dv + d, v);
	}
}

// Mean key / value (fp32) of block b (positions b * pool .. b * pool + pool - 1) of kv head g; the members are read back from
// the ring, as it holds them.
template <typename CT>
__device__ __forceinline__ void kv_pool_block(float *kp, float *vp, const CT *kc, const CT *vc, int b, int g, int dk, int dv, int ring, int pool,
                                              int max_blocks) {
	const float inv = 1.0f / (float)pool;
	for (int d = threadIdx.x; d < dk + dv; d += blockDim.x) {
		float s = 0.f;
		for (int t = 0; t < pool; ++t) {
			const int slot = (b * pool + t) % ring;
			s += d < dk ? cache_get(kc, ((size_t)g * ring + slot) * dk + d) : cache_get(vc, ((size_t)g * ring + slot) * dv + (d - dk));
		}
		if (d < dk) kp[((size_t)g * max_blocks + b) * dk + d] = s * inv;
		else vp[((size_t)g * max_blocks + b) * dv + (d - dk)] = s * inv;
	}
}

// x += rms(sum_j y_j) * (offset + w) for one row: y holds nsum partial outputs (part j at y + j * ldy) — the sum over a row's
// selected experts in slot order, or the single output of a dense sublayer.  ys: dim floats of shared memory.
__device__ __forceinline__ void norm_residual_row(float *x, const float *y, int ldy, int nsum, const float *w, float woff, float eps, int dim, float *ys,
                                                  float *red) {
	float ss = 0.f;
	for (int e = threadIdx.x; e < dim; e += blockDim.x) {
		float v = 0.f;
		for (int j = 0; j < nsum; ++j) v += __ldcg(y + (size_t)j * ldy + e);
		ys[e] = v;
		ss += v * v;
	}
	ss = block_sum(ss, red);
	const float r = 1.0f / sqrtf(ss / dim + eps);
	for (int e = threadIdx.x; e < dim; e += blockDim.x) x[e] += ys[e] * r * (woff + w[e]);
}

} // namespace stack
} // namespace yalm
