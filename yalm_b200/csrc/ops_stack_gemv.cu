// One-row products of the layered executor with what follows them fused in: the decode step's GEMVs.
//
// The product itself is the .yalm decode path's streaming GEMV (gemv.cuh: x staged in shared memory, every warp owns four
// output rows with sixteen 16-byte weight loads in flight per lane, persistent grid).  Around it:
//   head   the input may be a gated activation of a (gate | up) row: x[f] = act(g[f]) * (u[f] + offset), applied while staging;
//          or the token-shifted norm of a residual row: h = rms(x) w, input = h + (previous position's h - h) * mu, every CTA
//          recomputing the row's mean square, CTA 0 leaving h for the other sublayer
//   tail   the CTA that finishes last (a ticket from one atomic counter, after a device-scope fence) runs, on the complete
//          output vector, either the sublayer's output norm + residual add (x += rms(y) (offset + w)) or the q / k norm, value
//          blending, cache append and — when this position completes a block — the block's mean key / value; or the hand-over
//          of the row's h to the token-shift state (once every CTA has read the old one); or the residual add of a parallel
//          block, x += (this output + another sublayer's) + the selected experts' outputs.
// One launch instead of two to four, on the path where launches, not bytes, are the larger cost.
#include "common.cuh"

#include <cuda_bf16.h>

#include "gemv.cuh"
#include "launch.h"
#include "stack_rows.cuh"

namespace yalm {
namespace stack {

constexpr int kGemvThreads = 256;

struct GemvTailArgs {
	// product: out (d) = alpha * W (d, n) x (n)
	float *out;
	const float *x;
	const char *w;
	int n, d;
	float alpha;
	// head: glu == 1: x[f] = glu_value(x[f], x[n + f]) of a (gate | up) row of 2 n floats; glu == 2: x[f] = act_value(x[f]), no gate
	int glu, act;
	float act_alpha, limit, up_offset;
	// tail
	int tail; // 0 none, 1 norm + residual, 2 q / k norm + value blending + append (+ block mean)
	unsigned *counter;
	float *res;          // 1: the residual row (d)
	const float *nw;     // 1: norm weight
	const float *next_w; // 1, optional: the next sublayer's input norm, next_out = rms(res) next_w, from the finished residual row
	float *next_out;
	float woff, eps;
	void *kring, *vring; // 2
	float *vfirst, *kpool, *vpool;
	const float *qnorm, *knorm, *vmix;
	int vmode, nq, nk, nv, dk, dv, ring, pool, max_blocks, n_kv, cache_f32;
	int pos0;
	const int *ctl;
	// head 2 (norm + token shift): x is the residual row; hw its norm weight (one number if hscalar); mu the shift weight;
	// hstate the previous position's h (zero at position 0); hout receives this row's h.  Tail 3 then moves hout to hstate.
	int head, hscalar;
	const float *hw, *mu;
	float hwoff, heps;
	float *hstate, *hout;
	// tail 4: res += (out + add1) + sum_{j < nslots} slots[j * ldslots + .]
	const float *add1, *slots;
	int nslots, ldslots;
};

// R rows per warp, 16 / R chunks of each in flight: few output rows (d below the warps the GPU holds) take fewer rows per
// warp, so that every SM still streams.
template <int DT, int R>
__global__ void __launch_bounds__(kGemvThreads) gemv_tail_kernel(GemvTailArgs a) {
	extern __shared__ __align__(16) float smem[];
	__shared__ int is_last;
	float *red = smem, *xs = smem + 36;
	constexpr int EP = WTraits<DT>::EP, B = WTraits<DT>::BYTES, U = 16 / R;
	const int lane = threadIdx.x & 31;
	const int warps = (gridDim.x * blockDim.x) >> 5, gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
	const size_t row_bytes = (size_t)a.n * B;
	const int ntasks = (a.d + R - 1) / R;
	if (a.glu == 2) {
		for (int e = threadIdx.x * 4; e < a.n; e += blockDim.x * 4) {
			float4 v = *reinterpret_cast<const float4 *>(a.x + e);
			v.x = act_value(v.x, a.act), v.y = act_value(v.y, a.act), v.z = act_value(v.z, a.act), v.w = act_value(v.w, a.act);
			*reinterpret_cast<float4 *>(xs + xs_slot<EP>(e)) = v;
		}
	} else if (a.glu) {
		for (int e = threadIdx.x * 4; e < a.n; e += blockDim.x * 4) {
			const float4 g = *reinterpret_cast<const float4 *>(a.x + e), u = *reinterpret_cast<const float4 *>(a.x + a.n + e);
			float4 v;
			v.x = glu_value(g.x, u.x, a.act, a.act_alpha, a.limit, a.up_offset), v.y = glu_value(g.y, u.y, a.act, a.act_alpha, a.limit, a.up_offset);
			v.z = glu_value(g.z, u.z, a.act, a.act_alpha, a.limit, a.up_offset), v.w = glu_value(g.w, u.w, a.act, a.act_alpha, a.limit, a.up_offset);
			*reinterpret_cast<float4 *>(xs + xs_slot<EP>(e)) = v;
		}
	} else if (a.head == 2) {
		float ss = 0.f;
		for (int e = threadIdx.x * 4; e < a.n; e += blockDim.x * 4) {
			const float4 v = *reinterpret_cast<const float4 *>(a.x + e);
			ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
		}
		ss = block_sum(ss, red);
		const float r = 1.0f / sqrtf(ss / a.n + a.heps);
		const bool start = first_pos(a.ctl, a.pos0) == 0;
		for (int e = threadIdx.x * 4; e < a.n; e += blockDim.x * 4) {
			const float4 v = *reinterpret_cast<const float4 *>(a.x + e), m = *reinterpret_cast<const float4 *>(a.mu + e);
			const float4 pv = start ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4 *>(a.hstate + e);
			float4 g;
			if (a.hscalar) g.x = g.y = g.z = g.w = a.hwoff + a.hw[0];
			else g = make_float4(a.hwoff + a.hw[e], a.hwoff + a.hw[e + 1], a.hwoff + a.hw[e + 2], a.hwoff + a.hw[e + 3]);
			const float4 h = make_float4(v.x * r * g.x, v.y * r * g.y, v.z * r * g.z, v.w * r * g.w);
			const float4 o = make_float4(h.x + (pv.x - h.x) * m.x, h.y + (pv.y - h.y) * m.y, h.z + (pv.z - h.z) * m.z, h.w + (pv.w - h.w) * m.w);
			*reinterpret_cast<float4 *>(xs + xs_slot<EP>(e)) = o;
			if (blockIdx.x == 0) *reinterpret_cast<float4 *>(a.hout + e) = h;
		}
	} else
		stage_x_plain<EP>(xs, a.x, a.n);
	__syncthreads();
	for (int t = gw; t < ntasks; t += warps) {
		const int row = t * R;
		const char *rows[R];
#pragma unroll
		for (int r = 0; r < R; ++r) rows[r] = a.w + (size_t)min(row + r, a.d - 1) * row_bytes;
		float acc[R];
		warp_rows_dot<DT, R, U>(rows, xs, a.n, acc);
#pragma unroll
		for (int r = 0; r < R; ++r)
			if (lane == r && row + r < a.d) a.out[row + r] = a.alpha * acc[r];
	}
	if (!a.tail) return;
	// ---- tail: the last CTA to arrive sees every CTA's rows (fence, ticket, fence) ----
	__threadfence();
	__syncthreads();
	if (threadIdx.x == 0) is_last = atomicAdd(a.counter, 1u) == gridDim.x - 1;
	__syncthreads();
	if (!is_last) return;
	__threadfence();
	if (a.tail == 1) {
		norm_residual_row(a.res, a.out, 0, 1, a.nw, a.woff, a.eps, a.d, xs, red); // xs: free now, sized for max(n, d) by the launcher
		if (a.next_w) { // every thread reads back the elements it has just written
			float ss = 0.f;
			for (int e = threadIdx.x; e < a.d; e += blockDim.x) ss += a.res[e] * a.res[e];
			ss = block_sum(ss, red);
			const float r = 1.0f / sqrtf(ss / a.d + a.eps);
			for (int e = threadIdx.x; e < a.d; e += blockDim.x) a.next_out[e] = a.res[e] * r * a.next_w[e];
		}
	} else if (a.tail == 3) { // every CTA has staged its input from the old state
		for (int e = threadIdx.x; e < a.n; e += blockDim.x) a.hstate[e] = __ldcg(a.hout + e);
	} else if (a.tail == 4) {
		for (int e = threadIdx.x; e < a.d; e += blockDim.x) {
			const float v = a.add1 ? a.add1[e] + __ldcg(a.out + e) : __ldcg(a.out + e);
			float f = 0.f;
			for (int j = 0; j < a.nslots; ++j) f += a.slots[(size_t)j * a.ldslots + e];
			a.res[e] += v + f;
		}
	} else {
		const int p = first_pos(a.ctl, a.pos0), slot = p % a.ring;
		if (a.cache_f32) qkv_post_row<float>(a.out, (float *)a.kring, (float *)a.vring, a.vfirst, a.qnorm, a.knorm, a.vmix, a.vmode, a.nq, a.nk, a.nv, a.dk, a.dv, a.ring, slot, a.eps, red);
		else qkv_post_row<__nv_bfloat16>(a.out, (__nv_bfloat16 *)a.kring, (__nv_bfloat16 *)a.vring, a.vfirst, a.qnorm, a.knorm, a.vmix, a.vmode, a.nq, a.nk, a.nv, a.dk, a.dv, a.ring, slot, a.eps, red);
		if (a.pool > 0 && (p + 1) % a.pool == 0 && p / a.pool < a.max_blocks) { // this position completes block p / pool
			__syncthreads();                                                      // the row just appended is one of its members
			for (int g = 0; g < a.n_kv; ++g) {
				if (a.cache_f32) kv_pool_block<float>(a.kpool, a.vpool, (const float *)a.kring, (const float *)a.vring, p / a.pool, g, a.dk, a.dv, a.ring, a.pool, a.max_blocks);
				else kv_pool_block<__nv_bfloat16>(a.kpool, a.vpool, (const __nv_bfloat16 *)a.kring, (const __nv_bfloat16 *)a.vring, p / a.pool, g, a.dk, a.dv, a.ring, a.pool, a.max_blocks);
			}
		}
	}
	if (threadIdx.x == 0) *a.counter = 0; // ready for the next launch on this stream
}

static int launch_tail(const GemvTailArgs &a, int dtype, cudaStream_t st) {
	const int ep = dtype == YALM_F32 ? 4 : 8;
	if (!a.out || !a.x || !a.w || a.n < 1 || a.d < 1 || a.n % ep || ((uintptr_t)a.w & 15) || ((uintptr_t)a.x & 15) || (a.tail && !a.counter)) return YALM_EINVAL;
	const int ch = 32 * ep;
	const size_t xs = (size_t)std::max((a.n + ch - 1) / ch * ch, a.tail == 1 ? a.d : 0);
	const size_t smem = (36 + xs) * sizeof(float);
	if ((int)smem > device_info().max_smem_optin) return YALM_EINVAL;
	// rows per warp: 4 when that still gives every resident warp a task, else 2, else 1
	const long want = (long)device_info().sms * (kGemvThreads / 32) * 2;
	int rows = (a.d + 3) / 4 >= want ? 4 : (a.d + 1) / 2 >= want ? 2 : 1;
	while (rows < 4 && a.n / ch < 16 / rows) rows *= 2; // short rows: the 16 loads in flight must come from more rows
	cudaError_t err = cudaSuccess;
#define TAIL_LAUNCH(DT_, R_)                                                                                                          \
	do {                                                                                                                              \
		const int grid = persistent_grid((const void *)gemv_tail_kernel<DT_, R_>, kGemvThreads, smem, (a.d + R_ - 1) / R_, &err);    \
		if (err != cudaSuccess) return (int)err;                                                                                      \
		gemv_tail_kernel<DT_, R_><<<grid, kGemvThreads, smem, st>>>(a);                                                               \
	} while (0)
#define TAIL_ROWS(DT_)                                                                                                                \
	do {                                                                                                                              \
		if (rows == 4) TAIL_LAUNCH(DT_, 4);                                                                                           \
		else if (rows == 2) TAIL_LAUNCH(DT_, 2);                                                                                      \
		else TAIL_LAUNCH(DT_, 1);                                                                                                     \
	} while (0)
	if (dtype == YALM_F32) TAIL_ROWS(YALM_F32);
	else if (dtype == YALM_F16) TAIL_ROWS(YALM_F16);
	else if (dtype == YALM_BF16) TAIL_ROWS(YALM_BF16);
	else return YALM_EINVAL;
#undef TAIL_ROWS
#undef TAIL_LAUNCH
	return (int)cudaGetLastError();
}

} // namespace stack
} // namespace yalm

using namespace yalm::stack;

// YALM_STACK_TAIL=0: the same products with what follows them as separate launches (A/B of the last-CTA tails)
static bool tail_separate() {
	static const bool off = [] { const char *e = getenv("YALM_STACK_TAIL"); return e && e[0] == '0'; }();
	return off;
}

// res (d) += rms(y) * (w_offset + nw), y = W x (d rows, n columns; y is also left in `y`).  gu != 0: x is a (gate | up) row of
// 2 n floats and the product's input is act(g) * (u + up_offset) (yalm_glu_act_rows's arithmetic).  counter: a zeroed
// device word that the kernel leaves zero.
extern "C" int yalm_gemv_norm_residual(float *res, float *y, const float *x, const void *w, const float *nw, float w_offset, float eps, int n, int d,
                                       int dtype, int gu, int act, float act_alpha, float limit, float up_offset, unsigned *counter, yalm_stream_t s) {
	if (!res || !nw) return YALM_EINVAL;
	GemvTailArgs a{};
	a.out = y, a.x = x, a.w = (const char *)w, a.n = n, a.d = d, a.alpha = 1.f;
	a.glu = gu, a.act = act, a.act_alpha = act_alpha, a.limit = limit, a.up_offset = up_offset;
	a.tail = 1, a.counter = counter, a.res = res, a.nw = nw, a.woff = w_offset, a.eps = eps;
	if (tail_separate()) {
		a.tail = 0;
		const int rc = launch_tail(a, dtype, (cudaStream_t)s);
		return rc ? rc : yalm_norm_residual_rows(res, y, d, 1, nw, w_offset, eps, 1, d, s);
	}
	return launch_tail(a, dtype, (cudaStream_t)s);
}

// qkv (nq + nk + nv) = W x, then yalm_qkv_post_rows for this one row and, if the position completes a block of `pool`
// positions, that block's mean key / value (yalm_kv_pool_rows).
extern "C" int yalm_gemv_qkv_post(float *qkv, const float *x, const void *w, int n, int dtype, void *key_ring, void *value_ring, float *vfirst,
                                  const float *qnorm, const float *knorm, const float *vmix, int vmode, int n_heads, int n_kv, int dk, int dv, int ring,
                                  float eps, int cache_f32, float *key_pool, float *value_pool, int pool, int max_blocks, int pos0, const int *ctl,
                                  unsigned *counter, yalm_stream_t s) {
	if (!key_ring || !value_ring || ring < 1 || (vmode && !vfirst) || (vmode == 2 && !vmix) || (pool > 0 && (!key_pool || !value_pool))) return YALM_EINVAL;
	GemvTailArgs a{};
	a.nq = n_heads * dk, a.nk = n_kv * dk, a.nv = n_kv * dv;
	a.out = qkv, a.x = x, a.w = (const char *)w, a.n = n, a.d = a.nq + a.nk + a.nv, a.alpha = 1.f;
	a.tail = 2, a.counter = counter, a.kring = key_ring, a.vring = value_ring, a.vfirst = vfirst, a.kpool = key_pool, a.vpool = value_pool;
	a.qnorm = qnorm, a.knorm = knorm, a.vmix = vmix, a.vmode = vmode, a.dk = dk, a.dv = dv, a.ring = ring, a.pool = pool, a.max_blocks = max_blocks;
	a.n_kv = n_kv, a.cache_f32 = cache_f32, a.eps = eps, a.pos0 = pos0, a.ctl = ctl;
	if (tail_separate()) {
		a.tail = 0;
		int rc = launch_tail(a, dtype, (cudaStream_t)s);
		if (!rc) rc = yalm_qkv_post_rows(qkv, a.d, key_ring, value_ring, vfirst, a.nv, qnorm, knorm, vmix, vmode, 1, n_heads, n_kv, dk, dv, ring, eps, cache_f32, pos0, ctl, s);
		if (!rc && pool > 0) rc = yalm_kv_pool_rows(key_pool, value_pool, key_ring, value_ring, 1, n_kv, dk, dv, ring, pool, max_blocks, cache_f32, pos0, ctl, s);
		return rc;
	}
	return launch_tail(a, dtype, (cudaStream_t)s);
}

// One decode row of a parallel block's mixer input: out (d) = W (d, n) hs with h = rms(x) (w_offset + hw) (hw one number if
// scalar_weight), hs = h + (state - h) * shift (state: the previous position's h, zero at position 0); h is left in h_out
// and becomes the state.  yalm_norm_shift_rows + the product, as one launch.
extern "C" int yalm_gemv_norm_shift(float *out, const float *x, const void *w, int n, int d, int dtype, const float *hw, int scalar_weight, float w_offset,
                                    float eps, const float *shift, float *state, float *h_out, int pos0, const int *ctl, unsigned *counter, yalm_stream_t s) {
	if (!hw || !shift || !state || !h_out || ((uintptr_t)shift & 15) || ((uintptr_t)state & 15) || ((uintptr_t)h_out & 15) || (!scalar_weight && ((uintptr_t)hw & 15)))
		return YALM_EINVAL;
	GemvTailArgs a{};
	a.out = out, a.x = x, a.w = (const char *)w, a.n = n, a.d = d, a.alpha = 1.f;
	a.head = 2, a.hw = hw, a.hscalar = scalar_weight, a.hwoff = w_offset, a.heps = eps, a.mu = shift, a.hstate = state, a.hout = h_out;
	a.tail = 3, a.counter = counter, a.pos0 = pos0, a.ctl = ctl;
	return launch_tail(a, dtype, (cudaStream_t)s);
}

// The last product of a parallel block's decode row with the block's residual add as its tail: y = alpha W x, then
// res += (y + add1) + sum_{j < nslots} slots[j] (add1: another sublayer's output or null; slots: the selected experts' outputs).
extern "C" int yalm_gemv_residual_sum(float *res, float *y, const float *x, const void *w, float alpha, int n, int d, int dtype, const float *add1,
                                      const float *slots, int nslots, int ldslots, unsigned *counter, yalm_stream_t s) {
	if (!res || nslots < 0 || (nslots && !slots)) return YALM_EINVAL;
	GemvTailArgs a{};
	a.out = y, a.x = x, a.w = (const char *)w, a.n = n, a.d = d, a.alpha = alpha;
	a.tail = 4, a.counter = counter, a.res = res, a.add1 = add1, a.slots = slots, a.nslots = nslots, a.ldslots = ldslots;
	return launch_tail(a, dtype, (cudaStream_t)s);
}

// yalm_gemv_norm_residual with a plain activation on the input (act >= 0: x[f] = act(x[f]) while it is staged; yalm_act_rows'
// codes) and, optionally, the next sublayer's input norm from the finished residual row: next_out = rms(res) * next_w.
extern "C" int yalm_gemv_act_norm_residual_norm(float *res, float *y, const float *x, const void *w, const float *nw, float eps, int n, int d, int dtype, int act,
                                                const float *next_w, float *next_out, unsigned *counter, yalm_stream_t s) {
	if (!res || !nw || (next_w && !next_out)) return YALM_EINVAL;
	GemvTailArgs a{};
	a.out = y, a.x = x, a.w = (const char *)w, a.n = n, a.d = d, a.alpha = 1.f;
	a.glu = act >= 0 ? 2 : 0, a.act = act;
	a.tail = 1, a.counter = counter, a.res = res, a.nw = nw, a.woff = 0.f, a.eps = eps, a.next_w = next_w, a.next_out = next_out;
	if (tail_separate()) {
		a.tail = 0;
		int rc = launch_tail(a, dtype, (cudaStream_t)s);
		if (!rc) rc = yalm_norm_residual_rows(res, y, d, 1, nw, 0.f, eps, 1, d, s);
		if (!rc && next_w) rc = yalm_norm_shift_rows(next_out, nullptr, res, next_w, 0, 0.f, eps, nullptr, nullptr, 1, d, 0, nullptr, s);
		return rc;
	}
	return launch_tail(a, dtype, (cudaStream_t)s);
}
