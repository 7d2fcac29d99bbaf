// Windowed attention with pooled blocks for many query rows (a portion of a prompt) over the bf16 key / value rings, on the
// tensor cores.  Same visibility rule and the same single softmax as ops_stack.cu's attn_window_pool_kernel, which remains
// the route for decode-sized calls, the fp32 cache and other head sizes.
//
// grid (ceil(n / 64), heads), 4 warps x 16 query rows.  Key tiles of 64 go through shared memory, two buffers deep (cp.async
// brings tile t + 1 from the rings while tile t is multiplied): first the pooled blocks
// 0 .. nb(last row) - 1 (fp32 means, rounded to bf16 as they are staged), then the tokens lo(first row) .. last row from
// their ring slots.  S = Q K^T and O += P V on mma.sync.m16n8k16 (bf16 in, fp32 accumulate); scores, running max and sum,
// and the weights are fp32, the weights are rounded to bf16 only as the operand of P V.  Per row the mask is an interval
// of the tile's key indices: blocks [0, nb(i)) or tokens [lo(i), i].
#include "common.cuh"
#include "launch.h"
#include "stack_rows.cuh"

#include <cuda_bf16.h>

#include <algorithm>

namespace yalm {
namespace stack {

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
	asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
	asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
	             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
	             : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
	asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
	             : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
	             : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16 bytes global -> shared without passing through registers; valid false: the 16 bytes are zero-filled (src is not read)
__device__ __forceinline__ void cp_async16(void *smem, const void *gmem, bool valid) {
	asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem), "r"(valid ? 16 : 0) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf2(float a, float b) {
	const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
	return *reinterpret_cast<const uint32_t *>(&h);
}

template <int DK, int DV>
__global__ void __launch_bounds__(128) attn_window_pool_mma_kernel(float *__restrict__ out, int ldo, const float *__restrict__ q, int ldq,
                                                                   const __nv_bfloat16 *__restrict__ kc, const __nv_bfloat16 *__restrict__ vc,
                                                                   const float *__restrict__ kp, const float *__restrict__ vp, int n, int n_heads, int n_kv,
                                                                   int ring, int max_blocks, int window, int pool, float scale, int pos0,
                                                                   const int *__restrict__ ctl, const float *__restrict__ sink, int v_heads) {
	constexpr int LDK = DK + 8, LDV = DV + 8; // padded rows: 16 bytes of skew keep ldmatrix conflict-free
	constexpr int KS = DK / 16;               // k-steps of Q K^T
	constexpr int OT = DV / 8;                // 8-wide output tiles of P V
	extern __shared__ __align__(16) __nv_bfloat16 smb[];
	__nv_bfloat16 *Qs = smb, *Kbuf = Qs + 64 * LDK, *Vbuf = Kbuf + 2 * 64 * LDK; // two key and two value tiles: the next one loads while this one is used
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int h = blockIdx.y, g = h / (n_heads / n_kv), i0 = blockIdx.x * 64;
	const int p0 = ctl ? ctl[CTL_POS] : pos0;
	const int gv = g % v_heads; // key heads beyond the value heads (further maps over the same values) wrap around
	const __nv_bfloat16 *kbase = kc + (size_t)g * ring * DK, *vbase = vc + (size_t)gv * ring * DV;
	const float *kpb = kp ? kp + (size_t)g * max_blocks * DK : nullptr, *vpb = vp ? vp + (size_t)gv * max_blocks * DV : nullptr;
	// Q tile: fp32 -> bf16 (rows past n: zeros)
	for (int c = threadIdx.x; c < 64 * (DK / 4); c += 128) {
		const int r = c / (DK / 4), d = (c % (DK / 4)) * 4;
		float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
		if (i0 + r < n) v = *reinterpret_cast<const float4 *>(q + (size_t)(i0 + r) * ldq + (size_t)h * DK + d);
		uint2 pk;
		pk.x = pack_bf2(v.x, v.y), pk.y = pack_bf2(v.z, v.w);
		*reinterpret_cast<uint2 *>(Qs + r * LDK + d) = pk;
	}
	__syncthreads();
	uint32_t qf[KS][4];
	{
		const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, cofs = (lane >> 4) * 8;
#pragma unroll
		for (int ks = 0; ks < KS; ++ks) ldsm_x4(qf[ks], (uint32_t)__cvta_generic_to_shared(Qs + r * LDK + ks * 16 + cofs));
	}
	float o[OT][4];
#pragma unroll
	for (int t = 0; t < OT; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
	float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f; // rows lane / 4 and lane / 4 + 8 of the warp's 16
	const int rA = i0 + warp * 16 + (lane >> 2), rB = rA + 8;
	// positions (rows past n repeat the last valid row: finite values that are never stored)
	const int iA = p0 + min(rA, n - 1), iB = p0 + min(rB, n - 1);
	const int i_first = p0 + i0, i_last = p0 + min(i0 + 63, n - 1);
	auto lo_of = [&](int i) { return window > 0 ? max(0, i - window + 1) : 0; };
	auto nb_of = [&](int i) { return (window > 0 && pool > 0 && i - window + 1 >= pool) ? min((i - window + 1) / pool, max_blocks) : 0; };
	const int loA = lo_of(iA), loB = lo_of(iB), nbA = nb_of(iA), nbB = nb_of(iB);
	const int nb_max = nb_of(i_last), lo_min = lo_of(i_first);
	const int pooled_tiles = (nb_max + 63) / 64, token_tiles = (i_last - lo_min) / 64 + 1;
	const int n_tiles = pooled_tiles + token_tiles;
	// Tile tt into buffer tt & 1.  Ring slots go global -> shared with cp.async (16 bytes each; rows past the last position are
	// zero-filled by a source size of 0), pooled means are fp32 and pass through registers to be rounded.
	auto stage = [&](int tt) {
		const bool pooled = tt < pooled_tiles;
		const int base = pooled ? tt * 64 : lo_min + (tt - pooled_tiles) * 64;
		__nv_bfloat16 *Ks = Kbuf + (tt & 1) * 64 * LDK, *Vs = Vbuf + (tt & 1) * 64 * LDV;
		if (pooled) {
			for (int c = threadIdx.x; c < 64 * (DK / 8); c += 128) {
				const int r = c / (DK / 8), d = (c % (DK / 8)) * 8;
				uint4 pk = make_uint4(0, 0, 0, 0);
				if (base + r < nb_max) {
					const float4 a = *reinterpret_cast<const float4 *>(kpb + (size_t)(base + r) * DK + d), b = *reinterpret_cast<const float4 *>(kpb + (size_t)(base + r) * DK + d + 4);
					pk.x = pack_bf2(a.x, a.y), pk.y = pack_bf2(a.z, a.w), pk.z = pack_bf2(b.x, b.y), pk.w = pack_bf2(b.z, b.w);
				}
				*reinterpret_cast<uint4 *>(Ks + r * LDK + d) = pk;
			}
			for (int c = threadIdx.x; c < 64 * (DV / 8); c += 128) {
				const int r = c / (DV / 8), d = (c % (DV / 8)) * 8;
				uint4 pk = make_uint4(0, 0, 0, 0);
				if (base + r < nb_max) {
					const float4 a = *reinterpret_cast<const float4 *>(vpb + (size_t)(base + r) * DV + d), b = *reinterpret_cast<const float4 *>(vpb + (size_t)(base + r) * DV + d + 4);
					pk.x = pack_bf2(a.x, a.y), pk.y = pack_bf2(a.z, a.w), pk.z = pack_bf2(b.x, b.y), pk.w = pack_bf2(b.z, b.w);
				}
				*reinterpret_cast<uint4 *>(Vs + r * LDV + d) = pk;
			}
		} else {
			for (int c = threadIdx.x; c < 64 * (DK / 8); c += 128) {
				const int r = c / (DK / 8), d = (c % (DK / 8)) * 8;
				const bool in = base + r <= i_last;
				cp_async16(Ks + r * LDK + d, kbase + (size_t)((in ? base + r : i_last) % ring) * DK + d, in);
			}
			for (int c = threadIdx.x; c < 64 * (DV / 8); c += 128) {
				const int r = c / (DV / 8), d = (c % (DV / 8)) * 8;
				const bool in = base + r <= i_last;
				cp_async16(Vs + r * LDV + d, vbase + (size_t)((in ? base + r : i_last) % ring) * DV + d, in);
			}
		}
		asm volatile("cp.async.commit_group;" ::: "memory"); // one group per tile, empty for a pooled one
	};
	stage(0);
	for (int tt = 0; tt < n_tiles; ++tt) {
		const bool pooled = tt < pooled_tiles;
		const int base = pooled ? tt * 64 : lo_min + (tt - pooled_tiles) * 64; // index of the tile's first key: block or position
		const __nv_bfloat16 *Ks = Kbuf + (tt & 1) * 64 * LDK, *Vs = Vbuf + (tt & 1) * 64 * LDV;
		__syncthreads(); // tile tt - 1 is read: its buffer may take tile tt + 1
		if (tt + 1 < n_tiles) {
			stage(tt + 1);
			asm volatile("cp.async.wait_group 1;" ::: "memory"); // all but the group just committed: tile tt has landed
		} else
			asm volatile("cp.async.wait_group 0;" ::: "memory");
		__syncthreads();
		// ---- S = Q K^T: 8 key tiles of 8 ----
		float s[8][4];
#pragma unroll
		for (int t = 0; t < 8; ++t) s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.f;
		{
			const int kr = (lane & 7) + (lane >> 4) * 8, kcofs = ((lane >> 3) & 1) * 8;
#pragma unroll
			for (int ks = 0; ks < KS; ++ks)
#pragma unroll
				for (int t = 0; t < 8; t += 2) {
					uint32_t b[4];
					ldsm_x4(b, (uint32_t)__cvta_generic_to_shared(Ks + (t * 8 + kr) * LDK + ks * 16 + kcofs));
					mma_bf16(s[t], qf[ks], b[0], b[1]);
					mma_bf16(s[t + 1], qf[ks], b[2], b[3]);
				}
		}
		// ---- scale, interval mask, online softmax (fp32) ----
		const int minA = pooled ? 0 : loA, maxA = pooled ? nbA - 1 : iA, minB = pooled ? 0 : loB, maxB = pooled ? nbB - 1 : iB;
		float mxA = -INFINITY, mxB = -INFINITY;
#pragma unroll
		for (int t = 0; t < 8; ++t) {
			const int key = base + t * 8 + (lane & 3) * 2;
			s[t][0] = (key >= minA && key <= maxA) ? s[t][0] * scale : -INFINITY;
			s[t][1] = (key + 1 >= minA && key + 1 <= maxA) ? s[t][1] * scale : -INFINITY;
			s[t][2] = (key >= minB && key <= maxB) ? s[t][2] * scale : -INFINITY;
			s[t][3] = (key + 1 >= minB && key + 1 <= maxB) ? s[t][3] * scale : -INFINITY;
			mxA = fmaxf(mxA, fmaxf(s[t][0], s[t][1]));
			mxB = fmaxf(mxB, fmaxf(s[t][2], s[t][3]));
		}
		mxA = fmaxf(mxA, __shfl_xor_sync(kFull, mxA, 1)), mxA = fmaxf(mxA, __shfl_xor_sync(kFull, mxA, 2));
		mxB = fmaxf(mxB, __shfl_xor_sync(kFull, mxB, 1)), mxB = fmaxf(mxB, __shfl_xor_sync(kFull, mxB, 2));
		const float nA = fmaxf(m0, mxA), nB = fmaxf(m1, mxB);
		// a row may see nothing yet (its first visible key lies in a later tile): keep its state empty without producing NaNs
		const float eA = nA == -INFINITY ? 0.f : nA, eB = nB == -INFINITY ? 0.f : nB;
		const float cA = m0 == -INFINITY ? 0.f : expf(m0 - eA), cB = m1 == -INFINITY ? 0.f : expf(m1 - eB);
		m0 = nA, m1 = nB;
		l0 *= cA, l1 *= cB;
#pragma unroll
		for (int t = 0; t < OT; ++t) o[t][0] *= cA, o[t][1] *= cA, o[t][2] *= cB, o[t][3] *= cB;
		uint32_t pf[4][4]; // P as A fragments: key steps of 16
#pragma unroll
		for (int t = 0; t < 8; ++t) {
			const float p0v = expf(s[t][0] - eA), p1v = expf(s[t][1] - eA), p2v = expf(s[t][2] - eB), p3v = expf(s[t][3] - eB);
			l0 += p0v + p1v, l1 += p2v + p3v;
			pf[t >> 1][(t & 1) * 2] = pack_bf2(p0v, p1v);
			pf[t >> 1][(t & 1) * 2 + 1] = pack_bf2(p2v, p3v);
		}
		// ---- O += P V ----
		{
			const int vr = (lane & 7) + ((lane >> 3) & 1) * 8, vcofs = (lane >> 4) * 8;
#pragma unroll
			for (int kk = 0; kk < 4; ++kk)
#pragma unroll
				for (int t = 0; t < OT; t += 2) {
					uint32_t b[4];
					ldsm_x4_t(b, (uint32_t)__cvta_generic_to_shared(Vs + (kk * 16 + vr) * LDV + t * 8 + vcofs));
					mma_bf16(o[t], pf[kk], b[0], b[1]);
					mma_bf16(o[t + 1], pf[kk], b[2], b[3]);
				}
		}
	}
	l0 += __shfl_xor_sync(kFull, l0, 1), l0 += __shfl_xor_sync(kFull, l0, 2);
	l1 += __shfl_xor_sync(kFull, l1, 1), l1 += __shfl_xor_sync(kFull, l1, 2);
	const float f0 = stack::softmax_finish(m0, l0, sink, h), f1 = stack::softmax_finish(m1, l1, sink, h);
#pragma unroll
	for (int t = 0; t < OT; ++t) {
		const int d = h * DV + t * 8 + (lane & 3) * 2;
		if (rA < n) *reinterpret_cast<float2 *>(out + (size_t)rA * ldo + d) = make_float2(o[t][0] * f0, o[t][1] * f0);
		if (rB < n) *reinterpret_cast<float2 *>(out + (size_t)rB * ldo + d) = make_float2(o[t][2] * f1, o[t][3] * f1);
	}
}

template <int DK, int DV>
static int launch_mma(float *out, int ldo, const float *q, int ldq, const void *kr, const void *vr, const float *kp, const float *vp, int n, int n_heads,
                      int n_kv, int ring, int max_blocks, int window, int pool, float scale, int pos0, const int *ctl, const float *sink, int v_heads,
                      cudaStream_t st) {
	const size_t smem = sizeof(__nv_bfloat16) * (3 * 64 * (DK + 8) + 2 * 64 * (DV + 8)); // Q, two key tiles, two value tiles
	static bool configured = false;
	if (!configured && smem > 48 * 1024) {
		YALM_TRY(cudaFuncSetAttribute(attn_window_pool_mma_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
		configured = true;
	}
	attn_window_pool_mma_kernel<DK, DV><<<dim3((n + 63) / 64, n_heads), 128, smem, st>>>(out, ldo, q, ldq, (const __nv_bfloat16 *)kr, (const __nv_bfloat16 *)vr,
	                                                                                   kp, vp, n, n_heads, n_kv, ring, max_blocks, window, pool, scale, pos0,
	                                                                                   ctl, sink, v_heads);
	return (int)cudaGetLastError();
}


// ---- decode rows of latent attention on the tensor cores: the heads are the M tile -------------------------------------------
// Every head of a row reads the same cached rows [latent | rotated key part] (bf16, row stride ld), key = the row's dk channels,
// value = its first DV.  With the queries already mapped to the cached rows' space (ops_stack_latent.cu: latent_query_rows_kernel),
// 16 heads x dk is one A operand, a tile of 64 cached rows serves as B for the scores (as stored) and again, transposed by
// ldmatrix, for the weighted sums, so a cached row is fetched once per CTA for all heads.
//
// grid (ceil(heads / 16), rows, key splits), 4 warps.  Tiles of 64 keys go through two shared-memory buffers filled by cp.async.
// Warp w multiplies the 16 heads by keys 16 w .. 16 w + 15 of the tile over all of dk; the scores (fp32, scaled, masked past the
// row's position) meet in shared memory; every warp then runs the same online softmax over all 64 and accumulates P V for ITS
// quarter of the value channels.  One split: the row is finished here (sink included); more: unnormalised partials
// (accumulator, max, sum) in the layout attn_latent_merge_kernel joins.  Same visibility rule as attn_latent_rows_kernel:
// position i sees rows j with 0 <= i - j < window (0: all).  Queries and weights are rounded to bf16 as operands; scores, max, sum
// and accumulators are fp32.
template <int DV>
__global__ void __launch_bounds__(128) attn_latent_mma_rows_kernel(float *__restrict__ out, int ldo, const float *__restrict__ q, int ldq,
                                                                   const __nv_bfloat16 *__restrict__ rows, int ld, float *__restrict__ part, int n_heads,
                                                                   int dk, int ring, int window, float scale, int pos0, const int *__restrict__ ctl,
                                                                   const float *__restrict__ sink) {
	constexpr int DW = DV / 4, OT = DW / 8, LDS = 68; // value channels and 8-wide output tiles per warp; padded score rows
	extern __shared__ __align__(16) __nv_bfloat16 smb[];
	const int LDK = dk + 8;                       // padded rows: 16 bytes of skew keep ldmatrix conflict-free
	__nv_bfloat16 *Qs = smb, *Kbuf = Qs + 16 * LDK;
	float *Ss = reinterpret_cast<float *>(Kbuf + 2 * 64 * LDK);
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int h0 = blockIdx.x * 16, m = blockIdx.y, z = blockIdx.z, nsplit = gridDim.z;
	const int i = stack::first_pos(ctl, pos0) + m;
	const int lo = window > 0 ? max(0, i - window + 1) : 0;
	const int tiles = (i - lo) / 64 + 1, per = (tiles + nsplit - 1) / nsplit;
	const int t_begin = z * per, t_end = min(tiles, t_begin + per);
	// the 16 heads' queries as bf16 (heads past the last: zeros)
	for (int c = threadIdx.x; c < 16 * (dk / 4); c += 128) {
		const int r = c / (dk / 4), d = (c % (dk / 4)) * 4;
		float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
		if (h0 + r < n_heads) v = *reinterpret_cast<const float4 *>(q + (size_t)m * ldq + (size_t)(h0 + r) * dk + d);
		uint2 pk;
		pk.x = pack_bf2(v.x, v.y), pk.y = pack_bf2(v.z, v.w);
		*reinterpret_cast<uint2 *>(Qs + r * LDK + d) = pk;
	}
	auto stage = [&](int tt) { // tile tt (positions lo + 64 tt ..) into buffer tt & 1; rows past the position are zero-filled
		__nv_bfloat16 *Ks = Kbuf + (tt & 1) * 64 * LDK;
		const int base = lo + tt * 64, pieces = dk / 8;
		for (int c = threadIdx.x; c < 64 * pieces; c += 128) {
			const int r = c / pieces, d = (c % pieces) * 8;
			const bool in = base + r <= i;
			cp_async16(Ks + r * LDK + d, rows + (size_t)((in ? base + r : i) % ring) * ld + d, in);
		}
		asm volatile("cp.async.commit_group;" ::: "memory");
	};
	float o[OT][4];
#pragma unroll
	for (int t = 0; t < OT; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
	float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f; // heads lane / 4 and lane / 4 + 8 of the 16
	if (t_begin < t_end) stage(t_begin);
	for (int tt = t_begin; tt < t_end; ++tt) {
		const __nv_bfloat16 *Ks = Kbuf + (tt & 1) * 64 * LDK;
		__syncthreads(); // the previous tile's buffer and scores are read; the queries are in place
		if (tt + 1 < t_end) {
			stage(tt + 1);
			asm volatile("cp.async.wait_group 1;" ::: "memory");
		} else
			asm volatile("cp.async.wait_group 0;" ::: "memory");
		__syncthreads();
		// ---- scores of this warp's 16 keys ----
		{
			float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
			const int ar = (lane & 7) + ((lane >> 3) & 1) * 8, acofs = (lane >> 4) * 8;
			const int kr = (lane & 7) + (lane >> 4) * 8, kcofs = ((lane >> 3) & 1) * 8;
			for (int ks = 0; ks < dk / 16; ++ks) {
				uint32_t a[4], b[4];
				ldsm_x4(a, (uint32_t)__cvta_generic_to_shared(Qs + ar * LDK + ks * 16 + acofs));
				ldsm_x4(b, (uint32_t)__cvta_generic_to_shared(Ks + (warp * 16 + kr) * LDK + ks * 16 + kcofs));
				mma_bf16(s[0], a, b[0], b[1]);
				mma_bf16(s[1], a, b[2], b[3]);
			}
			const int base = lo + tt * 64 + warp * 16;
#pragma unroll
			for (int t = 0; t < 2; ++t) {
				const int col = warp * 16 + t * 8 + (lane & 3) * 2, key = base + t * 8 + (lane & 3) * 2;
				float *ra = Ss + (lane >> 2) * LDS + col, *rb = Ss + ((lane >> 2) + 8) * LDS + col;
				ra[0] = key <= i ? s[t][0] * scale : -INFINITY, ra[1] = key + 1 <= i ? s[t][1] * scale : -INFINITY;
				rb[0] = key <= i ? s[t][2] * scale : -INFINITY, rb[1] = key + 1 <= i ? s[t][3] * scale : -INFINITY;
			}
		}
		__syncthreads();
		// ---- online softmax over the tile's 64 keys (the same in every warp), then this warp's value channels ----
		float sa[8][2], sb[8][2], mxA = -INFINITY, mxB = -INFINITY;
#pragma unroll
		for (int t = 0; t < 8; ++t) {
			const float2 va = *reinterpret_cast<const float2 *>(Ss + (lane >> 2) * LDS + t * 8 + (lane & 3) * 2);
			const float2 vb = *reinterpret_cast<const float2 *>(Ss + ((lane >> 2) + 8) * LDS + t * 8 + (lane & 3) * 2);
			sa[t][0] = va.x, sa[t][1] = va.y, sb[t][0] = vb.x, sb[t][1] = vb.y;
			mxA = fmaxf(mxA, fmaxf(va.x, va.y)), mxB = fmaxf(mxB, fmaxf(vb.x, vb.y));
		}
		mxA = fmaxf(mxA, __shfl_xor_sync(kFull, mxA, 1)), mxA = fmaxf(mxA, __shfl_xor_sync(kFull, mxA, 2));
		mxB = fmaxf(mxB, __shfl_xor_sync(kFull, mxB, 1)), mxB = fmaxf(mxB, __shfl_xor_sync(kFull, mxB, 2));
		const float nA = fmaxf(m0, mxA), nB = fmaxf(m1, mxB); // finite: a tile holds at least one visible key
		const float cA = m0 == -INFINITY ? 0.f : expf(m0 - nA), cB = m1 == -INFINITY ? 0.f : expf(m1 - nB);
		m0 = nA, m1 = nB;
		l0 *= cA, l1 *= cB;
#pragma unroll
		for (int t = 0; t < OT; ++t) o[t][0] *= cA, o[t][1] *= cA, o[t][2] *= cB, o[t][3] *= cB;
		uint32_t pf[4][4]; // the weights as A fragments: key steps of 16
#pragma unroll
		for (int t = 0; t < 8; ++t) {
			const float p0v = expf(sa[t][0] - nA), p1v = expf(sa[t][1] - nA), p2v = expf(sb[t][0] - nB), p3v = expf(sb[t][1] - nB);
			l0 += p0v + p1v, l1 += p2v + p3v;
			pf[t >> 1][(t & 1) * 2] = pack_bf2(p0v, p1v);
			pf[t >> 1][(t & 1) * 2 + 1] = pack_bf2(p2v, p3v);
		}
		{
			const int vr = (lane & 7) + ((lane >> 3) & 1) * 8, vcofs = (lane >> 4) * 8;
#pragma unroll
			for (int kk = 0; kk < 4; ++kk)
#pragma unroll
				for (int t = 0; t < OT; t += 2) {
					uint32_t b[4];
					ldsm_x4_t(b, (uint32_t)__cvta_generic_to_shared(Ks + (kk * 16 + vr) * LDK + warp * DW + t * 8 + vcofs));
					mma_bf16(o[t], pf[kk], b[0], b[1]);
					mma_bf16(o[t + 1], pf[kk], b[2], b[3]);
				}
		}
	}
	l0 += __shfl_xor_sync(kFull, l0, 1), l0 += __shfl_xor_sync(kFull, l0, 2);
	l1 += __shfl_xor_sync(kFull, l1, 1), l1 += __shfl_xor_sync(kFull, l1, 2);
	const int hA = h0 + (lane >> 2), hB = hA + 8;
	if (part) {
		float *pa = part + ((size_t)(m * n_heads + hA) * nsplit + z) * (DV + 2), *pb = part + ((size_t)(m * n_heads + hB) * nsplit + z) * (DV + 2);
#pragma unroll
		for (int t = 0; t < OT; ++t) {
			const int d = warp * DW + t * 8 + (lane & 3) * 2;
			if (hA < n_heads) pa[d] = o[t][0], pa[d + 1] = o[t][1];
			if (hB < n_heads) pb[d] = o[t][2], pb[d + 1] = o[t][3];
		}
		if (warp == 0 && (lane & 3) == 0) {
			if (hA < n_heads) pa[DV] = m0, pa[DV + 1] = l0;
			if (hB < n_heads) pb[DV] = m1, pb[DV + 1] = l1;
		}
	} else {
		const float f0 = hA < n_heads ? stack::softmax_finish(m0, l0, sink, hA) : 0.f, f1 = hB < n_heads ? stack::softmax_finish(m1, l1, sink, hB) : 0.f;
#pragma unroll
		for (int t = 0; t < OT; ++t) {
			const int d = warp * DW + t * 8 + (lane & 3) * 2;
			if (hA < n_heads) out[(size_t)m * ldo + (size_t)hA * DV + d] = o[t][0] * f0, out[(size_t)m * ldo + (size_t)hA * DV + d + 1] = o[t][1] * f0;
			if (hB < n_heads) out[(size_t)m * ldo + (size_t)hB * DV + d] = o[t][2] * f1, out[(size_t)m * ldo + (size_t)hB * DV + d + 1] = o[t][3] * f1;
		}
	}
}

template <int DV>
static int launch_latent_mma(float *out, int ldo, const float *q, int ldq, const void *rows, int ld, float *part, int n, int n_heads, int dk, int ring,
                             int window, float scale, int nsplit, int pos0, const int *ctl, const float *sink, size_t smem, cudaStream_t st) {
	if (smem > 48 * 1024) YALM_TRY(cudaFuncSetAttribute(attn_latent_mma_rows_kernel<DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
	attn_latent_mma_rows_kernel<DV><<<dim3((n_heads + 15) / 16, n, nsplit), 128, smem, st>>>(out, ldo, q, ldq, (const __nv_bfloat16 *)rows, ld, part, n_heads, dk,
	                                                                                       ring, window, scale, pos0, ctl, sink);
	return (int)cudaGetLastError();
}


// ---- sigmoid-weighted attention whose values are its keys, many rows, tensor cores ------------------------------------------
// Same rule as ops_stack_state.cu's attn_sigmoid_rows_kernel (the route for decode-sized calls, the fp32 ring and other head
// sizes): row i sees the positions lo(i) .. i from the ring and 0 .. min(keep, lo(i)) - 1 from the kept-first buffer, with
// weight sigmoid(q . k * scale + rel[bucket[i - j], h] + hb[h]), not normalised; out = (sum of weight * key) * sigmoid(gate).
// Same tiling as above, but one tile buffer pair serves both products (S = Q K^T reads the tile's rows, O += P K reads it
// transposed), there is no running maximum or sum, and the distance bias of this head comes from a shared-memory table
// over the distances the CTA meets inside the window (tb entries; farther ones, met only through kept tokens, are looked
// up in global memory).
template <int D>
__global__ void __launch_bounds__(128) attn_sigmoid_mma_kernel(float *__restrict__ out, int ldo, const float *__restrict__ q, int ldq,
                                                               const __nv_bfloat16 *__restrict__ ring_buf, const __nv_bfloat16 *__restrict__ first_buf,
                                                               const float *__restrict__ gate, int ldg, const float *__restrict__ rel,
                                                               const int *__restrict__ bucket, const float *__restrict__ hb,
                                                               const float *__restrict__ table, int ldt, int n, int n_heads, int n_kv, int ring, int window,
                                                               int keep, float scale, int tb, int pos0, const int *__restrict__ ctl) {
	constexpr int LD = D + 8, KS = D / 16, OT = D / 8;
	extern __shared__ __align__(16) __nv_bfloat16 smb[];
	__nv_bfloat16 *Qs = smb, *Kbuf = Qs + 64 * LD;
	float *relt = reinterpret_cast<float *>(Kbuf + 2 * 64 * LD);
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int h = blockIdx.y, g = h / (n_heads / n_kv), i0 = blockIdx.x * 64;
	const int p0 = ctl ? ctl[CTL_POS] : pos0;
	const __nv_bfloat16 *rbase = ring_buf + (size_t)g * ring * D, *fbase = first_buf ? first_buf + (size_t)g * keep * D : nullptr;
	const float hbh = hb ? hb[h] : 0.f;
	for (int c = threadIdx.x; c < 64 * (D / 4); c += 128) {
		const int r = c / (D / 4), d = (c % (D / 4)) * 4;
		float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
		if (i0 + r < n) v = *reinterpret_cast<const float4 *>(q + (size_t)(i0 + r) * ldq + (size_t)h * D + d);
		uint2 pk;
		pk.x = pack_bf2(v.x, v.y), pk.y = pack_bf2(v.z, v.w);
		*reinterpret_cast<uint2 *>(Qs + r * LD + d) = pk;
	}
	const int i_first = p0 + i0, i_last = p0 + min(i0 + 63, n - 1);
	auto lo_of = [&](int i) { return window > 0 ? max(0, i - window + 1) : 0; };
	const int lo_min = lo_of(i_first);
	const int nfirst_max = min(keep, lo_of(i_last));
	// table (optional): the same bias per (head, distance), rel[bucket[d], h] + hb[h], laid out for one coalesced read
	const float *trow = table ? table + (size_t)h * ldt : nullptr;
	for (int d = threadIdx.x; d < tb; d += 128)
		relt[d] = d > i_last ? hbh : trow ? trow[d] : rel ? rel[(size_t)bucket[d] * n_heads + h] + hbh : hbh;
	__syncthreads();
	auto bias_far = [&](int dist) { return trow ? trow[dist] : rel ? rel[(size_t)bucket[dist] * n_heads + h] + hbh : hbh; };
	const bool table_covers = i_last - lo_min < tb; // every distance inside the window of this CTA's rows is in the table
	uint32_t qf[KS][4];
	{
		const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, cofs = (lane >> 4) * 8;
#pragma unroll
		for (int ks = 0; ks < KS; ++ks) ldsm_x4(qf[ks], (uint32_t)__cvta_generic_to_shared(Qs + r * LD + ks * 16 + cofs));
	}
	float o[OT][4];
#pragma unroll
	for (int t = 0; t < OT; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
	const int rA = i0 + warp * 16 + (lane >> 2), rB = rA + 8;
	const int iA = p0 + min(rA, n - 1), iB = p0 + min(rB, n - 1); // rows past n repeat the last valid row and are never stored
	const int loA = lo_of(iA), loB = lo_of(iB), nfA = min(keep, loA), nfB = min(keep, loB);
	const int first_tiles = (nfirst_max + 63) / 64, token_tiles = (i_last - lo_min) / 64 + 1;
	const int n_tiles = first_tiles + token_tiles;
	auto stage = [&](int tt) {
		const bool first = tt < first_tiles;
		const int base = first ? tt * 64 : lo_min + (tt - first_tiles) * 64;
		__nv_bfloat16 *Ks = Kbuf + (tt & 1) * 64 * LD;
		for (int c = threadIdx.x; c < 64 * (D / 8); c += 128) {
			const int r = c / (D / 8), d = (c % (D / 8)) * 8;
			if (first) {
				const bool in = base + r < nfirst_max;
				cp_async16(Ks + r * LD + d, fbase + (size_t)(in ? base + r : 0) * D + d, in);
			} else {
				const bool in = base + r <= i_last;
				cp_async16(Ks + r * LD + d, rbase + (size_t)((in ? base + r : i_last) % ring) * D + d, in);
			}
		}
		asm volatile("cp.async.commit_group;" ::: "memory");
	};
	stage(0);
	for (int tt = 0; tt < n_tiles; ++tt) {
		const bool first = tt < first_tiles;
		const int base = first ? tt * 64 : lo_min + (tt - first_tiles) * 64; // position of the tile's first key
		const __nv_bfloat16 *Ks = Kbuf + (tt & 1) * 64 * LD;
		__syncthreads();
		if (tt + 1 < n_tiles) {
			stage(tt + 1);
			asm volatile("cp.async.wait_group 1;" ::: "memory");
		} else
			asm volatile("cp.async.wait_group 0;" ::: "memory");
		__syncthreads();
		float s[8][4];
#pragma unroll
		for (int t = 0; t < 8; ++t) s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.f;
		{
			const int kr = (lane & 7) + (lane >> 4) * 8, kcofs = ((lane >> 3) & 1) * 8;
#pragma unroll
			for (int ks = 0; ks < KS; ++ks)
#pragma unroll
				for (int t = 0; t < 8; t += 2) {
					uint32_t b[4];
					ldsm_x4(b, (uint32_t)__cvta_generic_to_shared(Ks + (t * 8 + kr) * LD + ks * 16 + kcofs));
					mma_bf16(s[t], qf[ks], b[0], b[1]);
					mma_bf16(s[t + 1], qf[ks], b[2], b[3]);
				}
		}
		// ---- weights: an interval of positions per row, fp32 sigmoid ----
		const int minA = first ? 0 : loA, maxA = first ? nfA - 1 : iA, minB = first ? 0 : loB, maxB = first ? nfB - 1 : iB;
		// One stage at a time over all 32 scores of the lane, in place: every stage is a batch of independent instructions
		// (an element-by-element chain of table read, exponential and reciprocal leaves one warp per scheduler waiting).
		const bool from_table = !first && table_covers; // uniform: ring tiles read the shared-memory table without a branch
#pragma unroll
		for (int t = 0; t < 8; ++t) {
			const int key = base + t * 8 + (lane & 3) * 2;
#pragma unroll
			for (int e = 0; e < 4; ++e) {
				const int kk = key + (e & 1), i = e < 2 ? iA : iB;
				float b;
				if (from_table) b = relt[min(max(i - kk, 0), tb - 1)];
				else b = (kk >= (e < 2 ? minA : minB) && kk <= (e < 2 ? maxA : maxB)) ? bias_far(i - kk) : 0.f;
				s[t][e] = -(s[t][e] * scale + b);
			}
		}
		// fast exponential and reciprocal: the weight is rounded to bf16 as the operand of the second product
#pragma unroll
		for (int t = 0; t < 8; ++t)
#pragma unroll
			for (int e = 0; e < 4; ++e) s[t][e] = __expf(s[t][e]);
#pragma unroll
		for (int t = 0; t < 8; ++t)
#pragma unroll
			for (int e = 0; e < 4; ++e) s[t][e] = __fdividef(1.0f, 1.0f + s[t][e]);
		uint32_t pf[4][4];
#pragma unroll
		for (int t = 0; t < 8; ++t) {
			const int key = base + t * 8 + (lane & 3) * 2;
			const float w0 = (key >= minA && key <= maxA) ? s[t][0] : 0.f, w1 = (key + 1 >= minA && key + 1 <= maxA) ? s[t][1] : 0.f;
			const float w2 = (key >= minB && key <= maxB) ? s[t][2] : 0.f, w3 = (key + 1 >= minB && key + 1 <= maxB) ? s[t][3] : 0.f;
			pf[t >> 1][(t & 1) * 2] = pack_bf2(w0, w1);
			pf[t >> 1][(t & 1) * 2 + 1] = pack_bf2(w2, w3);
		}
		// ---- O += P K ----
		{
			const int vr = (lane & 7) + ((lane >> 3) & 1) * 8, vcofs = (lane >> 4) * 8;
#pragma unroll
			for (int kk = 0; kk < 4; ++kk)
#pragma unroll
				for (int t = 0; t < OT; t += 2) {
					uint32_t b[4];
					ldsm_x4_t(b, (uint32_t)__cvta_generic_to_shared(Ks + (kk * 16 + vr) * LD + t * 8 + vcofs));
					mma_bf16(o[t], pf[kk], b[0], b[1]);
					mma_bf16(o[t + 1], pf[kk], b[2], b[3]);
				}
		}
	}
	// the output gate (raw values, 8-byte aligned pairs): all reads first, then the sigmoids
	float2 gA[OT], gB[OT];
#pragma unroll
	for (int t = 0; t < OT; ++t) {
		const int d = h * D + t * 8 + (lane & 3) * 2;
		gA[t] = (gate && rA < n) ? *reinterpret_cast<const float2 *>(gate + (size_t)rA * ldg + d) : make_float2(0.f, 0.f);
		gB[t] = (gate && rB < n) ? *reinterpret_cast<const float2 *>(gate + (size_t)rB * ldg + d) : make_float2(0.f, 0.f);
	}
#pragma unroll
	for (int t = 0; t < OT; ++t) {
		const int d = h * D + t * 8 + (lane & 3) * 2;
		if (gate) {
			o[t][0] *= __fdividef(1.0f, 1.0f + __expf(-gA[t].x)), o[t][1] *= __fdividef(1.0f, 1.0f + __expf(-gA[t].y));
			o[t][2] *= __fdividef(1.0f, 1.0f + __expf(-gB[t].x)), o[t][3] *= __fdividef(1.0f, 1.0f + __expf(-gB[t].y));
		}
		if (rA < n) *reinterpret_cast<float2 *>(out + (size_t)rA * ldo + d) = make_float2(o[t][0], o[t][1]);
		if (rB < n) *reinterpret_cast<float2 *>(out + (size_t)rB * ldo + d) = make_float2(o[t][2], o[t][3]);
	}
}

template <int D>
static int launch_sigmoid_mma(float *out, int ldo, const float *q, int ldq, const void *ring_buf, const void *first_buf, const float *gate, int ldg,
                              const float *rel, const int *bucket, const float *hb, const float *table, int ldt, int n, int n_heads, int n_kv, int ring,
                              int window, int keep, float scale, int context, int pos0, const int *ctl, cudaStream_t st) {
	const int tb = std::min(4096, window > 0 ? window + 64 : std::max(64, context));
	const size_t smem = sizeof(__nv_bfloat16) * (3 * 64 * (D + 8)) + sizeof(float) * tb;
	static size_t configured = 0;
	if (smem > 48 * 1024 && smem > configured) {
		YALM_TRY(cudaFuncSetAttribute(attn_sigmoid_mma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
		configured = smem;
	}
	attn_sigmoid_mma_kernel<D><<<dim3((n + 63) / 64, n_heads), 128, smem, st>>>(out, ldo, q, ldq, (const __nv_bfloat16 *)ring_buf,
	                                                                            (const __nv_bfloat16 *)first_buf, gate, ldg, rel, bucket, hb, table, ldt, n, n_heads,
	                                                                            n_kv, ring, window, keep, scale, tb, pos0, ctl);
	return (int)cudaGetLastError();
}

} // namespace stack
} // namespace yalm

using namespace yalm::stack;

// 1 when yalm_attn_window_pool_mma has a kernel for these head sizes (bf16 rings only).
extern "C" int yalm_attn_window_pool_mma_shape(int dk, int dv) {
	return (dk == 64 || dk == 128) && (dv == 32 || dv == 64 || dv == 128);
}

// The tensor-core route of yalm_attn_window_pool: bf16 key / value rings, head sizes of yalm_attn_window_pool_mma_shape,
// q rows and out rows 16-byte aligned (ldq, ldo multiples of 4 floats).
extern "C" int yalm_attn_window_pool_mma(float *out, int ldo, const float *q, int ldq, const void *key_ring, const void *value_ring,
                                         const float *key_pool, const float *value_pool, int n, int n_heads, int n_kv, int dk, int dv, int ring,
                                         int max_blocks, int window, int pool, float scale, int pos0, const int *ctl, yalm_stream_t s) {
	return yalm_attn_window_pool_mma_sink(out, ldo, q, ldq, key_ring, value_ring, key_pool, value_pool, n, n_heads, n_kv, dk, dv, ring, max_blocks, window,
	                                      pool, scale, pos0, ctl, nullptr, n_kv, s);
}

// The same with a sink per query head in the softmax's denominator (null: none) and v_heads value heads for n_kv key heads
// (key head g reads value head g % v_heads).
extern "C" int yalm_attn_window_pool_mma_sink(float *out, int ldo, const float *q, int ldq, const void *key_ring, const void *value_ring,
                                              const float *key_pool, const float *value_pool, int n, int n_heads, int n_kv, int dk, int dv, int ring,
                                              int max_blocks, int window, int pool, float scale, int pos0, const int *ctl, const float *sink, int v_heads,
                                              yalm_stream_t s) {
	if (v_heads < 1 || n_kv % v_heads) return YALM_EINVAL;
	if (!out || !q || !key_ring || !value_ring || n < 1 || n_kv < 1 || n_heads % n_kv || (pool > 0 && (!key_pool || !value_pool)) || ldq % 4 || ldo % 2 ||
	    ((uintptr_t)q & 15) || ((uintptr_t)out & 7) || !yalm_attn_window_pool_mma_shape(dk, dv))
		return YALM_EINVAL;
	cudaStream_t st = (cudaStream_t)s;
#define MMA_CASE(DK_, DV_)                                                                                                            \
	if (dk == DK_ && dv == DV_)                                                                                                       \
	return launch_mma<DK_, DV_>(out, ldo, q, ldq, key_ring, value_ring, key_pool, value_pool, n, n_heads, n_kv, ring, max_blocks, window, pool, scale, pos0, \
	                            ctl, sink, v_heads, st)
	MMA_CASE(64, 32);
	MMA_CASE(64, 64);
	MMA_CASE(64, 128);
	MMA_CASE(128, 32);
	MMA_CASE(128, 64);
	MMA_CASE(128, 128);
#undef MMA_CASE
	return YALM_EINVAL;
}

// 1 when yalm_attn_latent_mma_rows has a kernel for these sizes: key size a multiple of 16 whose two tile buffers fit into shared
// memory, value size 64, 128, 256 or 512 (at most the key size), row stride a multiple of 8.
static size_t latent_mma_smem(int dk) { return sizeof(__nv_bfloat16) * (size_t)(16 + 2 * 64) * (dk + 8) + sizeof(float) * 16 * 68; }
extern "C" int yalm_attn_latent_mma_shape(int dk, int dv, int ld) {
	return dk >= 16 && dk % 16 == 0 && (dv == 64 || dv == 128 || dv == 256 || dv == 512) && dv <= dk && ld >= dk && ld % 8 == 0 &&
	       (int)latent_mma_smem(dk) <= yalm::device_info().max_smem_optin;
}

// The tensor-core route of yalm_attn_latent_rows_sink for decode-sized calls: q (n, n_heads dk) fp32 already in the cached rows'
// space, rows bf16 (16-byte aligned).  nsplit: how many CTAs share a row's keys (1 ... 128; workspace as for yalm_attn_latent_rows
// when above 1), chosen by the caller from shapes alone.
extern "C" int yalm_attn_latent_mma_rows(float *out, int ldo, const float *q, int ldq, const void *rows, int ld, float *workspace, int n, int n_heads, int dk,
                                         int dv, int ring, int window, float scale, int nsplit, int pos0, const int *ctl, const float *sink, yalm_stream_t s) {
	if (!out || !q || !rows || n < 1 || n_heads < 1 || ring < 1 || nsplit < 1 || nsplit > 128 || (nsplit > 1 && !workspace) || !yalm_attn_latent_mma_shape(dk, dv, ld) ||
	    ((uintptr_t)rows & 15) || ((uintptr_t)q & 15) || ldq % 4 || (long)n * n_heads * nsplit > 4096)
		return YALM_EINVAL;
	cudaStream_t st = (cudaStream_t)s;
	const size_t smem = latent_mma_smem(dk);
	float *part = nsplit > 1 ? workspace : nullptr;
	int rc;
	if (dv == 64) rc = launch_latent_mma<64>(out, ldo, q, ldq, rows, ld, part, n, n_heads, dk, ring, window, scale, nsplit, pos0, ctl, sink, smem, st);
	else if (dv == 128) rc = launch_latent_mma<128>(out, ldo, q, ldq, rows, ld, part, n, n_heads, dk, ring, window, scale, nsplit, pos0, ctl, sink, smem, st);
	else if (dv == 256) rc = launch_latent_mma<256>(out, ldo, q, ldq, rows, ld, part, n, n_heads, dk, ring, window, scale, nsplit, pos0, ctl, sink, smem, st);
	else rc = launch_latent_mma<512>(out, ldo, q, ldq, rows, ld, part, n, n_heads, dk, ring, window, scale, nsplit, pos0, ctl, sink, smem, st);
	if (rc || nsplit == 1) return rc;
	return yalm_attn_latent_merge(out, ldo, workspace, n, n_heads, dv, nsplit, sink, s);
}

// 1 when yalm_attn_sigmoid_mma has a kernel for this head size (bf16 ring only).
extern "C" int yalm_attn_sigmoid_mma_shape(int dk) {
	return dk == 32 || dk == 64 || dk == 128;
}

// The tensor-core route of yalm_attn_sigmoid_rows: bf16 ring and kept-first buffer, head sizes of yalm_attn_sigmoid_mma_shape,
// q rows 16-byte aligned (ldq a multiple of 4 floats), out and gate rows 8-byte aligned.  table (optional, (n_heads, ldt) with
// ldt >= the most positions a sequence reaches): rel[bucket[d], h] + hb[h] per head and distance, read instead of rel / bucket / hb.
extern "C" int yalm_attn_sigmoid_mma(float *out, int ldo, const float *q, int ldq, const void *ring_buf, const void *first_buf, const float *gate, int ldg,
                                     const float *rel, const int *bucket, const float *hb, const float *table, int ldt, int n, int n_heads, int n_kv,
                                     int dk, int ring, int window, int keep, float scale, int context, int pos0, const int *ctl, yalm_stream_t s) {
	if (!out || !q || !ring_buf || n < 1 || n_kv < 1 || n_heads % n_kv || (keep > 0 && !first_buf) || (rel && !bucket) || ldq % 4 || ldo % 2 ||
	    ((uintptr_t)q & 15) || ((uintptr_t)out & 7) || (gate && (ldg % 2 || ((uintptr_t)gate & 7))) || !yalm_attn_sigmoid_mma_shape(dk))
		return YALM_EINVAL;
	cudaStream_t st = (cudaStream_t)s;
	if (dk == 32) return launch_sigmoid_mma<32>(out, ldo, q, ldq, ring_buf, first_buf, gate, ldg, rel, bucket, hb, table, ldt, n, n_heads, n_kv, ring, window, keep, scale, context, pos0, ctl, st);
	if (dk == 64) return launch_sigmoid_mma<64>(out, ldo, q, ldq, ring_buf, first_buf, gate, ldg, rel, bucket, hb, table, ldt, n, n_heads, n_kv, ring, window, keep, scale, context, pos0, ctl, st);
	return launch_sigmoid_mma<128>(out, ldo, q, ldq, ring_buf, first_buf, gate, ldg, rel, bucket, hb, table, ldt, n, n_heads, n_kv, ring, window, keep, scale, context, pos0, ctl, st);
}
