// The layered executor: Model's path for architectures described by a StackSpec (arch.h) — a list of layers, each with
// its own token mixer and feed-forward kind and sizes — where the reference has one homogeneous block (src/model.h:193-301).
// It shares the rest of the library with the .yalm models: the checkpoint container and loader (one device arena, pinned
// staging), InferenceState (stream, control block, logits, samplers), Model::forward / forward_batch / generate and the C
// ABI above them.  One pass takes n consecutive positions; n = 1 is a decode step (token and position may come from the
// device control block, so that sampling loops never leave the device), larger n is a portion of a prompt.
//
// Cache (owned by the model, like the reference's per-block key_cache / value_cache, src/model.h:238-240): per layer a
// key ring and a value ring of `ring` slots (slot = position % ring; ring = window + chunk capacity for windowed layers
// instead of the whole context, because a token that has left every window and whose block mean is taken is dead), plus,
// for pooled layers, one fp32 mean key / value per completed block of tokens.  A sequence restarts at position 0 and may
// only advance: the rings cannot seek.  Layers with other state (previous rows, convolution tails, matrix states, a ring of
// latent rows that all heads — and possibly several layers — read) list it in StackLayer::state_allocs; it is taken from the
// same arena.
#include "arch.h"
#include "loader.h"
#include "yalm_api.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>

// YALM_STACK_TRACE=1: a failing step names itself on stderr
static bool st_trace() {
	static const bool on = [] { const char *e = getenv("YALM_STACK_TRACE"); return e && e[0] == '1'; }();
	return on;
}
#define ST_TRY(x)                                                                                                                  \
	do {                                                                                                                           \
		int rc__ = (int)(x);                                                                                                       \
		if (rc__ != 0) {                                                                                                           \
			if (st_trace()) fprintf(stderr, "yalm_b200: %s:%d: %s -> %d\n", __FILE__, __LINE__, #x, rc__);                         \
			return rc__;                                                                                                           \
		}                                                                                                                          \
	} while (0)

namespace yalm {

struct StackLayer {
	LayerSpec spec;
	// device
	void *wqkv = nullptr, *wo = nullptr;     // (nq + nk + nv, dim), (dim, heads * vdim)
	float *qnorm = nullptr, *knorm = nullptr, *vmix = nullptr, *norm1 = nullptr, *norm2 = nullptr;
	void *wgu = nullptr, *wdown = nullptr;   // dense: (2 ff, dim) gate rows then up rows, (dim, ff)
	void *wg = nullptr, *wu = nullptr;       // experts stacked: (E, ff, dim) each; wdown then is (E, dim, ff)
	void *router = nullptr;                  // (E, dim)
	void *kring = nullptr, *vring = nullptr; // (kv heads, ring, dim | vdim), fp32 or bf16
	float *kpool = nullptr, *vpool = nullptr; // (kv heads, max_blocks, dim | vdim)
	int ring = 0, max_blocks = 0;
	int vmode = 0;                           // 0 plain values, 1 the first blending layer, 2 a later one
	// ---- parallel blocks: one packed projection of the mixer's input, then per-mixer pieces ----
	void *wproj = nullptr;                   // (proj_width, dim); columns in the order of the o_* offsets below
	float *shift = nullptr;                  // token-shift weight (dim)
	float *conv_w = nullptr, *conv_b = nullptr; // short convolution (channels, taps) [+ bias]
	// state-space mixer: columns [z | x | B | C | dt]
	float *dt_bias = nullptr, *a_log = nullptr, *skip = nullptr, *mix_norm = nullptr;
	void *wout = nullptr;                    // state-space / delta-rule output projection
	// sigmoid attention: columns [q | k | gate]
	int o_q = 0, o_k = 0, o_gate = 0;
	float *qkb = nullptr;                    // q bias then k bias
	float *rel = nullptr, *head_bias = nullptr;
	int *bucket = nullptr;                   // distance -> row of rel, max_seq_len entries
	float *bias_table = nullptr;             // (heads, max_seq_len): rel[bucket[d], h] + head_bias[h], what the tensor-core kernel stages
	void *kfirst = nullptr;                  // (kv heads, keep_first, dim): the kept first tokens' keys
	// delta rule: columns [q | k | v | beta | decay stage 1 | gate stage 1]
	int o_dq = 0, o_beta = 0, o_a1 = 0, o_g1 = 0;
	void *wa2 = nullptr, *wg2 = nullptr;     // second stages (heads * dim, rank), (heads * vdim, rank)
	float *d_a_log = nullptr, *d_dt_bias = nullptr, *d_norm = nullptr;
	// per-sequence state, fp32
	float *hprev = nullptr;                  // the previous position's normed input (dim)
	float *conv_state = nullptr;             // (channels, taps - 1)
	float *scan_state = nullptr;             // (heads, vdim, state | dim)
	std::vector<std::pair<void **, size_t>> state_allocs; // device buffers beside the rings, taken from the arena
	// ---- pre-norm layers with an input convolution and a weighted sum over depth ----
	float *inconv1 = nullptr, *inconv2 = nullptr;             // (dim, taps) each
	float *inconv1_state = nullptr, *inconv2_state = nullptr; // (taps - 1, dim): the sublayer's last normed inputs
	float *depth_w = nullptr;                                 // (layer + 2)
	// latent attention: columns [query latent | key / value latent + shared key part (own cache only) | gate]
	int o_kv = 0, kv_owner = -1;                              // kv_owner: the layer whose ring this layer reads (itself, or kv_from)
	void *wuq = nullptr, *wuk = nullptr, *wuv = nullptr;      // (heads (dim + rot), q_rank), (heads dim, kv_rank), (heads vdim, kv_rank)
	void *wukt = nullptr;                                     // (heads, kv_rank, dim): every head's W_uk transposed, for the queries against cached rows
	float *rot_freq = nullptr;                                // rotary frequencies (rot dims / 2)
	float rot_mag = 1.f;
	// gated linear attention: columns [q | k | v | gate | decay stage 1]; wa2, d_dt_bias (the decay's bias), mix_norm, scan_state as above
	int o_v = 0;
	// experts: the choice bias; the shared expert
	float *router_bias = nullptr;
	void *wsgu = nullptr, *wsdown = nullptr;                  // (2 shared_ff, dim), (dim, shared_ff)
	// ---- layers with a norm before and after every sublayer ----
	bool sandwich = false;
	float *norm1b = nullptr, *norm2b = nullptr;               // the norms on the sublayers' outputs
	float *sink = nullptr;                                    // latent attention: one number per head in the softmax's denominator
	// differential attention: columns [q: map, head | k: map, kv head | v | one gate number per head]; kring holds maps * kv heads key
	// vectors per slot, vring kv heads; kpool / vpool (max_blocks = keep_first entries) the window's kept first tokens
	float lambda = 0.f;
	void *side_gate = nullptr, *side_proj = nullptr;          // token side input: (token_side, dim), (dim, token_side)
	float *side_norm = nullptr;
};

} // namespace yalm

using yalm::FfnSpec;
using yalm::LayerSpec;
using yalm::StackLayer;
using yalm::StackSpec;
using yalm::TensorRole;

// ------------------------------------------------------------------------------------------------------------------------
// Config
// ------------------------------------------------------------------------------------------------------------------------
int Config::from_json(YALMData &data, int context, int compute) {
	yalm::JValue j;
	if (!yalm::json_parse(data.config_json.data(), data.config_json.size(), &j) || !j.is_object()) {
		fprintf(stderr, "yalm_b200: config.json is not a JSON object\n");
		return YALM_EFORMAT;
	}
	const std::string name = j["architecture"].string_or("");
	const yalm::ArchEntry *a = yalm::find_arch(name);
	if (!a) {
		fprintf(stderr, "yalm_b200: unknown architecture '%s' (registered: %s)\n", name.c_str(), yalm::arch_names().c_str());
		return YALM_EFORMAT;
	}
	const int rc = a->configure(j, *this);
	if (rc) return rc;
	StackSpec &s = *stack;
	for (int i = 0; i < (int)s.layers.size(); ++i) { // sizes that only the tensors give
		yalm::LayerSpec &l = s.layers[i];
		auto rows = [&](TensorRole role) {
			const Tensor *t = data.find(s.tensor_name(i, role, -1));
			return t ? t->shape[0] : 0;
		};
		if (l.kind == yalm::MixerKind::Parallel) {
			l.delta.decay_rank = rows(TensorRole::DeltaDecay1), l.delta.gate_rank = rows(TensorRole::DeltaGate1);
			if (l.delta.decay_rank < 1 || l.delta.gate_rank < 1) {
				fprintf(stderr, "yalm_b200: layer %d: the delta rule's two-stage projections are missing\n", i);
				return YALM_EFORMAT;
			}
		}
		if (l.kind == yalm::MixerKind::LinearAttention && (l.gla.decay_rank = rows(TensorRole::GlaDecay1)) < 1) {
			fprintf(stderr, "yalm_b200: layer %d: the decay's two-stage projection is missing\n", i);
			return YALM_EFORMAT;
		}
		if (l.mix.rel_rows > 0 && (l.mix.rel_rows = rows(TensorRole::RelBias)) < 2) {
			fprintf(stderr, "yalm_b200: layer %d: the distance-bias table needs at least two rows\n", i);
			return YALM_EFORMAT;
		}
	}
	const Tensor *emb = data.find(s.tensor_name(0, TensorRole::Embed, -1));
	if (!emb) {
		fprintf(stderr, "yalm_b200: the checkpoint has no embedding tensor\n");
		return YALM_EFORMAT;
	}
	weight_dtype = compute >= 0 ? static_cast<DType>(compute) : emb->dtype;
	if (weight_dtype != DType::F32 && weight_dtype != DType::F16 && weight_dtype != DType::BF16) {
		fprintf(stderr, "yalm_b200: layered models compute in F32, F16 or BF16\n");
		return YALM_EFORMAT;
	}
	// learned positions bound the context
	if (context > 0) max_seq_len = s.learned_positions ? std::min(context, s.max_positions) : context;
	if (const char *e = getenv("YALM_STACK_CHUNK")) stack_chunk = std::max(1, atoi(e));
	return 0;
}

// ------------------------------------------------------------------------------------------------------------------------
// Loading
// ------------------------------------------------------------------------------------------------------------------------
namespace {

float widen(const void *p, size_t i, DType dt) {
	if (dt == DType::F32) return static_cast<const float *>(p)[i];
	const uint16_t u = static_cast<const uint16_t *>(p)[i];
	if (dt == DType::BF16) {
		const uint32_t w = (uint32_t)u << 16;
		float f;
		memcpy(&f, &w, 4);
		return f;
	}
	// fp16
	const uint32_t sign = (u >> 15) & 1, ex = (u >> 10) & 31, man = u & 1023;
	uint32_t w;
	if (ex == 0) {
		if (man == 0) w = sign << 31;
		else {
			int e = -1;
			uint32_t m = man;
			do { ++e; m <<= 1; } while (!(m & 1024));
			w = (sign << 31) | ((uint32_t)(127 - 15 - e) << 23) | ((m & 1023) << 13);
		}
	} else if (ex == 31) w = (sign << 31) | 0x7f800000u | (man << 13);
	else w = (sign << 31) | ((ex + 112) << 23) | (man << 13);
	float f;
	memcpy(&f, &w, 4);
	return f;
}

uint16_t narrow_bf16(float f) { // round to nearest even
	uint32_t w;
	memcpy(&w, &f, 4);
	if ((w & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((w >> 16) | 0x40);
	w += 0x7fffu + ((w >> 16) & 1);
	return (uint16_t)(w >> 16);
}

[[noreturn]] void die(const std::string &msg) {
	std::cerr << "FATAL: " << msg << std::endl;
	abort();
}

} // namespace

// Host bytes of tensor `t` in dtype `want` (the tensor's own bytes when it already is; else converted into a buffer the
// model keeps until the upload).  Supported: anything -> F32, F32 -> BF16.
static const void *host_as(std::vector<std::vector<char>> &keep, const Tensor *t, DType want, size_t numel) {
	if (t->dtype == want) return t->data;
	if (t->dtype != DType::F32 && t->dtype != DType::F16 && t->dtype != DType::BF16) die("tensor " + t->name + ": unsupported dtype " + dtype_to_string(t->dtype));
	keep.emplace_back(numel * dtype_size(want));
	char *dst = keep.back().data();
	if (want == DType::F32) {
		float *o = reinterpret_cast<float *>(dst);
		for (size_t i = 0; i < numel; ++i) o[i] = widen(t->data, i, t->dtype);
	} else if (want == DType::BF16) {
		uint16_t *o = reinterpret_cast<uint16_t *>(dst);
		for (size_t i = 0; i < numel; ++i) o[i] = narrow_bf16(widen(t->data, i, t->dtype));
	} else
		die("tensor " + t->name + ": no conversion " + dtype_to_string(t->dtype) + " -> " + dtype_to_string(want));
	return dst;
}

namespace {
// one device destination assembled from host parts laid one after the other
struct Placement {
	void **slot;
	std::vector<std::pair<const void *, size_t>> parts;
	size_t bytes() const {
		size_t n = 0;
		for (auto &p : parts) n += p.second;
		return n;
	}
};
} // namespace

struct Model::StackScratch {
	int cap = 0;
	char *arena = nullptr;
	float *x = nullptr, *qkv = nullptr, *vfirst = nullptr, *att = nullptr, *y = nullptr, *gu = nullptr, *h = nullptr, *wts = nullptr, *xn = nullptr,
	      *logits = nullptr, *probs = nullptr;
	void *a16 = nullptr, *a16e = nullptr, *a16r = nullptr; // 16-bit operands of the tensor-core products: main stream, experts' stream, second mixer's stream
	float *hs = nullptr, *conv = nullptr, *aux = nullptr, *scan = nullptr, *att2 = nullptr, *y1 = nullptr, *y2 = nullptr; // parallel blocks
	float *hsh = nullptr;     // the shared expert's hidden rows (the routed experts' are in h)
	float *hist = nullptr;    // weighted sum over depth: the embedding output and every layer's result of the current rows, (layers + 1, cap, width)
	void *lat16 = nullptr, *lat_ek = nullptr, *lat_ev = nullptr; // latent attention, prompt portions: latents of the visible rows (bf16), keys / values per head
	float *latkv = nullptr;
	float *attn_ws = nullptr; // split partials of decode-sized attention calls
	int *ids = nullptr, *tokens = nullptr, *want = nullptr, *targets = nullptr;
	float *moe_gu = nullptr, *moe_ys = nullptr; // experts on the tensor cores: (gate | up) and down outputs of the slots sorted by expert
	int *order = nullptr;                       // slot at every place of that order
	unsigned *ticket = nullptr; // arrival counter of the one-row products with a fused tail (zero between launches)
	int hist_slabs = 0;
	bool xn_valid = false;    // xn already holds the next sublayer's normed input (left there by the previous product's tail)
	std::vector<Placement> placements; // filled by build_stack, consumed by cuda_stack
	// decode rows of a parallel block: its independent sublayers (experts, the second mixer) run on side streams that fork from and
	// join the caller's stream through these events; inside a captured step they become parallel branches of the graph
	cudaStream_t side[2] = {nullptr, nullptr};
	cudaEvent_t fork[2] = {nullptr, nullptr}, join[2] = {nullptr, nullptr};
	~StackScratch() {
		for (int i = 0; i < 2; ++i) {
			if (side[i]) cudaStreamDestroy(side[i]);
			if (fork[i]) cudaEventDestroy(fork[i]);
			if (join[i]) cudaEventDestroy(join[i]);
		}
		cudaFree(arena);
	}
};

void Model::build_stack(YALMData &data) {
	const Config &c = *config;
	const StackSpec &s = *c.stack;
	const DType dt = c.weight_dtype;
	_scratch = std::make_shared<StackScratch>();
	std::vector<Placement> &pl = _scratch->placements;
	auto tensor = [&](int layer, TensorRole role, int expert, std::initializer_list<int> shape) -> const Tensor * {
		const std::string name = s.tensor_name(layer, role, expert);
		const Tensor *t = data.find(name);
		if (!t) die("missing tensor: " + name);
		size_t i = 0;
		for (int d : shape) {
			if (t->shape[i] != d) die("tensor " + name + ": unexpected shape");
			++i;
		}
		for (; i < 4; ++i)
			if (t->shape[i] != 0) die("tensor " + name + ": unexpected rank");
		return t;
	};
	auto mat = [&](const Tensor *t) { return std::make_pair(host_as(_host_converted, t, dt, t->size / dtype_size(t->dtype)), t->size / dtype_size(t->dtype) * dtype_size(dt)); };
	auto vec32 = [&](const Tensor *t) { return std::make_pair(host_as(_host_converted, t, DType::F32, t->size / dtype_size(t->dtype)), t->size / dtype_size(t->dtype) * 4); };

	pl.push_back({&token_embedding_table, {mat(tensor(0, TensorRole::Embed, -1, {s.vocab, s.width}))}});
	if (s.learned_positions) pl.push_back({&_pos_table, {mat(tensor(0, TensorRole::Positions, -1, {s.max_positions, s.width}))}});
	pl.push_back({(void **)&rms_final_weight, {vec32(s.norm_scalar ? tensor(0, TensorRole::FinalNorm, -1, {}) : tensor(0, TensorRole::FinalNorm, -1, {s.width}))}});
	if (s.token_side > 0) pl.push_back({&_side_table, {mat(tensor(0, TensorRole::SideEmbed, -1, {s.vocab, s.token_side * (int)s.layers.size()}))}});
	if (s.depth_average) _scratch->hist_slabs = (int)s.layers.size() + 1;
	if (s.embed_norm) pl.push_back({(void **)&_embed_norm, {vec32(s.norm_scalar ? tensor(0, TensorRole::EmbedNorm, -1, {}) : tensor(0, TensorRole::EmbedNorm, -1, {s.width}))}});
	pl.push_back({&wcls, {mat(tensor(0, TensorRole::Head, -1, {s.vocab, s.width}))}});
	// latent attention's tensors, rotary table and cache ring (layers with their own W_dkv); the packed projection's parts go to `proj`
	auto load_latent = [&](int i, std::shared_ptr<StackLayer> &L, Placement &proj, int W) {
		const yalm::LayerSpec &ls = L->spec;
		const yalm::MixerSpec &m = ls.mix;
		const yalm::LatentSpec &a = ls.latent;
		const int no = m.heads * m.vdim, row = a.kv_rank + a.rot_dim;
		const bool own = a.kv_from < 0;
		const int nq = m.heads * (m.dim + a.rot_dim), qcols = a.q_rank > 0 ? a.q_rank : nq; // q_rank 0: the queries themselves
		L->o_q = 0, L->o_kv = qcols, L->o_gate = qcols + (own ? row : 0);
		L->kv_owner = own ? i : a.kv_from;
		proj.parts.push_back(mat(a.q_rank > 0 ? tensor(i, TensorRole::LatentDq, -1, {a.q_rank, W}) : tensor(i, TensorRole::Wq, -1, {nq, W})));
		if (own) proj.parts.push_back(mat(tensor(i, TensorRole::LatentDkv, -1, {row, W})));
		if (m.out_gate) proj.parts.push_back(mat(tensor(i, TensorRole::OutGate, -1, {no, W})));
		if (a.q_rank > 0) pl.push_back({(void **)&L->qnorm, {vec32(tensor(i, TensorRole::LatentDqNorm, -1, {a.q_rank}))}});
		if (own) pl.push_back({(void **)&L->knorm, {vec32(tensor(i, TensorRole::LatentDkvNorm, -1, {a.kv_rank}))}});
		if (a.q_rank > 0) pl.push_back({&L->wuq, {mat(tensor(i, TensorRole::LatentUq, -1, {nq, a.q_rank}))}});
		if (m.sink) pl.push_back({(void **)&L->sink, {vec32(tensor(i, TensorRole::Sink, -1, {m.heads}))}});
		// W_uk then W_uv in one piece: prompt portions multiply the cached latents by both at once
		if (m.dim > 0)
			pl.push_back({&L->wuk, {mat(tensor(i, TensorRole::LatentUk, -1, {m.heads * m.dim, a.kv_rank})), mat(tensor(i, TensorRole::LatentUv, -1, {no, a.kv_rank}))}});
		else
			pl.push_back({&L->wuv, {mat(tensor(i, TensorRole::LatentUv, -1, {no, a.kv_rank}))}});
		if (m.dim > 0) { // the same matrix, each head transposed: an output channel of W_uk^T q is then one contiguous row
			const auto uk = mat(tensor(i, TensorRole::LatentUk, -1, {m.heads * m.dim, a.kv_rank}));
			const size_t es = dtype_size(dt);
			_host_converted.emplace_back(uk.second);
			char *t = _host_converted.back().data();
			const char *src = static_cast<const char *>(uk.first);
			for (int hh = 0; hh < m.heads; ++hh)
				for (int d = 0; d < m.dim; ++d)
					for (int cc = 0; cc < a.kv_rank; ++cc)
						memcpy(t + (((size_t)hh * a.kv_rank + cc) * m.dim + d) * es, src + (((size_t)hh * m.dim + d) * a.kv_rank + cc) * es, es);
			pl.push_back({&L->wukt, {{t, uk.second}}});
		}
		pl.push_back({&L->wo, {mat(tensor(i, TensorRole::Wo, -1, {W, no}))}});
		if (a.rot.dims > 0) {
			std::vector<float> fr;
			a.rot.table(&fr, &L->rot_mag);
			_host_converted.emplace_back(fr.size() * sizeof(float));
			memcpy(_host_converted.back().data(), fr.data(), fr.size() * sizeof(float));
			pl.push_back({(void **)&L->rot_freq, {{_host_converted.back().data(), fr.size() * sizeof(float)}}});
		}
		if (own) {
			// one cache row [latent | rotated key part] per position; the ring covers the widest window of the layers that read it
			int span = m.window;
			bool unbounded = m.window == 0;
			for (int k = i + 1; k < (int)s.layers.size(); ++k)
				if (s.layers[k].kind == yalm::MixerKind::LatentAttention && s.layers[k].latent.kv_from == i)
					span = std::max(span, s.layers[k].mix.window), unbounded = unbounded || s.layers[k].mix.window == 0;
			L->ring = unbounded ? c.max_seq_len : std::min(c.max_seq_len, (span + c.stack_chunk + 63) / 64 * 64);
			const size_t cb = c.weight_dtype == DType::F32 ? 4 : 2;
			L->state_allocs.push_back({&L->kring, (size_t)L->ring * row * cb});
		}
		if (a.kv_rank > 512) die("latent attention: latents above 512 channels are not built");
	};
	bool have_first = false;
	for (int i = 0; i < (int)s.layers.size(); ++i) {
		auto L = std::make_shared<StackLayer>();
		L->spec = s.layers[i];
		const yalm::MixerSpec &m = L->spec.mix;
		if (s.parallel_block) {
			// ---- one norm, a packed projection of the mixer's input, per-mixer pieces, experts ----
			const int W = s.width;
			const yalm::LayerSpec &ls = L->spec;
			pl.push_back({(void **)&L->norm1, {vec32(s.norm_scalar ? tensor(i, TensorRole::Norm1, -1, {}) : tensor(i, TensorRole::Norm1, -1, {W}))}});
			if (s.token_shift) {
				pl.push_back({(void **)&L->shift, {vec32(tensor(i, TensorRole::Shift, -1, {W}))}});
				L->state_allocs.push_back({(void **)&L->hprev, (size_t)W * 4});
			}
			Placement proj{&L->wproj, {}};
			if (ls.kind == yalm::MixerKind::StateSpace) {
				const yalm::SsmSpec &q = ls.ssm;
				const int C = q.conv_channels(), inner = q.inner();
				proj.parts.push_back(mat(tensor(i, TensorRole::SsmIn, -1, {q.proj(), W})));
				pl.push_back({(void **)&L->conv_w, {vec32(tensor(i, TensorRole::SsmConv, -1, {C, q.conv}))}});
				pl.push_back({(void **)&L->conv_b, {vec32(tensor(i, TensorRole::SsmConvBias, -1, {C}))}});
				pl.push_back({(void **)&L->dt_bias, {vec32(tensor(i, TensorRole::SsmDtBias, -1, {q.heads}))}});
				pl.push_back({(void **)&L->a_log, {vec32(tensor(i, TensorRole::SsmALog, -1, {q.heads}))}});
				pl.push_back({(void **)&L->skip, {vec32(tensor(i, TensorRole::SsmD, -1, {q.heads}))}});
				pl.push_back({(void **)&L->mix_norm, {vec32(tensor(i, TensorRole::SsmNorm, -1, {inner}))}});
				pl.push_back({&L->wout, {mat(tensor(i, TensorRole::SsmOut, -1, {W, inner}))}});
				if (q.conv > 1) L->state_allocs.push_back({(void **)&L->conv_state, (size_t)C * (q.conv - 1) * 4});
				L->state_allocs.push_back({(void **)&L->scan_state, (size_t)q.heads * q.vdim * q.state * 4});
				if (q.state > 256) die("state-space mixer: state sizes above 256 are not built");
			} else if (ls.kind == yalm::MixerKind::Parallel) {
				const yalm::DeltaSpec &d = ls.delta;
				const int nq = m.heads * m.dim, nk = m.kv_heads * m.dim, no = m.heads * m.vdim;
				const int dk = d.kv_heads * d.dim, dv = d.heads * d.vdim, dg = d.heads * d.dim;
				L->o_q = 0, L->o_k = nq, L->o_gate = nq + nk;
				L->o_dq = L->o_gate + no, L->o_beta = L->o_dq + 2 * dk + dv, L->o_a1 = L->o_beta + d.heads, L->o_g1 = L->o_a1 + d.decay_rank;
				proj.parts.push_back(mat(tensor(i, TensorRole::Wq, -1, {nq, W})));
				proj.parts.push_back(mat(tensor(i, TensorRole::Wk, -1, {nk, W})));
				proj.parts.push_back(mat(tensor(i, TensorRole::OutGate, -1, {no, W})));
				proj.parts.push_back(mat(tensor(i, TensorRole::DeltaQ, -1, {dk, W})));
				proj.parts.push_back(mat(tensor(i, TensorRole::DeltaK, -1, {dk, W})));
				proj.parts.push_back(mat(tensor(i, TensorRole::DeltaV, -1, {dv, W})));
				proj.parts.push_back(mat(tensor(i, TensorRole::DeltaBeta, -1, {d.heads, W})));
				proj.parts.push_back(mat(tensor(i, TensorRole::DeltaDecay1, -1, {d.decay_rank, W})));
				proj.parts.push_back(mat(tensor(i, TensorRole::DeltaGate1, -1, {d.gate_rank, W})));
				pl.push_back({(void **)&L->qkb, {vec32(tensor(i, TensorRole::QBias, -1, {nq})), vec32(tensor(i, TensorRole::KBias, -1, {nk}))}});
				pl.push_back({(void **)&L->rel, {vec32(tensor(i, TensorRole::RelBias, -1, {m.rel_rows, m.heads}))}});
				pl.push_back({(void **)&L->head_bias, {vec32(tensor(i, TensorRole::HeadBias, -1, {m.heads}))}});
				pl.push_back({&L->wo, {mat(tensor(i, TensorRole::Wo, -1, {W, no}))}});
				{ // distance -> table row: exact below rows / 2, logarithmic up to rel_far, then the last row
					const int rows = m.rel_rows, half = rows / 2;
					if (m.rel_far <= half) die("distance bias: the farthest bucketed distance must exceed half the table");
					_host_converted.emplace_back((size_t)c.max_seq_len * sizeof(int));
					int *b = reinterpret_cast<int *>(_host_converted.back().data());
					for (int n = 0; n < c.max_seq_len; ++n)
						b[n] = n < half ? n
						                : std::min(rows - 1, half + (int)std::floor(std::log((double)n / half) / std::log((double)m.rel_far / half) * (rows - half)));
					pl.push_back({(void **)&L->bucket, {{b, (size_t)c.max_seq_len * sizeof(int)}}});
					const float *rel32 = static_cast<const float *>(vec32(tensor(i, TensorRole::RelBias, -1, {m.rel_rows, m.heads})).first);
					const float *hb32 = static_cast<const float *>(vec32(tensor(i, TensorRole::HeadBias, -1, {m.heads})).first);
					_host_converted.emplace_back((size_t)m.heads * c.max_seq_len * sizeof(float));
					float *tb = reinterpret_cast<float *>(_host_converted.back().data());
					for (int hh = 0; hh < m.heads; ++hh)
						for (int n = 0; n < c.max_seq_len; ++n) tb[(size_t)hh * c.max_seq_len + n] = rel32[(size_t)b[n] * m.heads + hh] + hb32[hh];
					pl.push_back({(void **)&L->bias_table, {{tb, (size_t)m.heads * c.max_seq_len * sizeof(float)}}});
				}
				pl.push_back({(void **)&L->conv_w, {vec32(tensor(i, TensorRole::DeltaQConv, -1, {dk, d.conv})), vec32(tensor(i, TensorRole::DeltaKConv, -1, {dk, d.conv})),
				                                    vec32(tensor(i, TensorRole::DeltaVConv, -1, {dv, d.conv}))}});
				pl.push_back({(void **)&L->d_a_log, {vec32(tensor(i, TensorRole::DeltaALog, -1, {d.heads}))}});
				pl.push_back({(void **)&L->d_dt_bias, {vec32(tensor(i, TensorRole::DeltaDtBias, -1, {dg}))}});
				pl.push_back({(void **)&L->d_norm, {vec32(tensor(i, TensorRole::DeltaNorm, -1, {d.vdim}))}});
				pl.push_back({&L->wa2, {mat(tensor(i, TensorRole::DeltaDecay2, -1, {dg, d.decay_rank}))}});
				pl.push_back({&L->wg2, {mat(tensor(i, TensorRole::DeltaGate2, -1, {dv, d.gate_rank}))}});
				pl.push_back({&L->wout, {mat(tensor(i, TensorRole::DeltaOut, -1, {W, dv}))}});
				if (d.conv > 1) L->state_allocs.push_back({(void **)&L->conv_state, (size_t)(2 * dk + dv) * (d.conv - 1) * 4});
				L->state_allocs.push_back({(void **)&L->scan_state, (size_t)d.heads * d.vdim * d.dim * 4});
				if (d.dim > 256 || m.dim > 256) die("parallel mixer: head sizes above 256 are not built");
				// the attention's keys (also its values): a ring for the window, a buffer for the kept first tokens
				L->ring = m.window > 0 ? std::min(c.max_seq_len, (m.window + c.stack_chunk + 63) / 64 * 64) : c.max_seq_len;
				const size_t cb = c.weight_dtype == DType::F32 ? 4 : 2;
				L->state_allocs.push_back({&L->kring, (size_t)m.kv_heads * L->ring * m.dim * cb});
				if (m.window > 0 && m.keep_first > 0) L->state_allocs.push_back({&L->kfirst, (size_t)m.kv_heads * m.keep_first * m.dim * cb});
			} else
				die("parallel blocks take a state-space or a parallel mixer");
			pl.push_back(proj);
			const FfnSpec &f = ls.ffn;
			if (f.kind == FfnSpec::Moe) {
				Placement g{&L->wg, {}}, u{&L->wu, {}}, dn{&L->wdown, {}};
				for (int e = 0; e < f.experts; ++e) {
					g.parts.push_back(mat(tensor(i, TensorRole::Gate, e, {f.ff, W})));
					u.parts.push_back(mat(tensor(i, TensorRole::Up, e, {f.ff, W})));
					dn.parts.push_back(mat(tensor(i, TensorRole::Down, e, {W, f.ff})));
				}
				pl.push_back(g), pl.push_back(u), pl.push_back(dn);
				pl.push_back({&L->router, {mat(tensor(i, TensorRole::Router, -1, {f.experts, W}))}});
			} else if (f.kind != FfnSpec::None)
				die("parallel blocks take experts or no feed-forward");
			_stack.push_back(L);
			continue;
		}
		if (s.sandwich_norm) {
			// ---- a norm before and after each sublayer, one packed projection of the mixer's input, a plain feed-forward, the token side input ----
			const int W = s.width;
			const yalm::LayerSpec &ls = L->spec;
			const FfnSpec &f = ls.ffn;
			L->sandwich = true;
			pl.push_back({(void **)&L->norm1, {vec32(tensor(i, TensorRole::Norm1, -1, {W}))}});
			pl.push_back({(void **)&L->norm1b, {vec32(tensor(i, TensorRole::Norm1Post, -1, {W}))}});
			Placement proj{&L->wproj, {}};
			if (ls.kind == yalm::MixerKind::LatentAttention) {
				load_latent(i, L, proj, W);
			} else if (ls.kind == yalm::MixerKind::Attention && m.maps == 2) {
				const int nq = m.maps * m.heads * m.dim, nk = m.maps * m.kv_heads * m.dim, nv = m.kv_heads * m.vdim, no = m.heads * m.vdim;
				L->o_q = 0, L->o_k = nq, L->o_v = nq + nk, L->o_gate = nq + nk + nv;
				// the checkpoint lays q and k out head by head as [map 1 | map 2]; the rows are reordered map by map, so that (map, head)
				// is one list of attention heads over (map, kv head) key heads and kv heads value heads
				auto by_map = [&](const Tensor *t, int heads) {
					const auto src = mat(t);
					const size_t rb = (size_t)W * dtype_size(dt) * m.dim; // bytes of one head's map
					_host_converted.emplace_back(src.second);
					char *dst = _host_converted.back().data();
					for (int mp = 0; mp < m.maps; ++mp)
						for (int hh = 0; hh < heads; ++hh)
							memcpy(dst + ((size_t)mp * heads + hh) * rb, static_cast<const char *>(src.first) + ((size_t)hh * m.maps + mp) * rb, rb);
					return std::make_pair((const void *)dst, src.second);
				};
				proj.parts.push_back(by_map(tensor(i, TensorRole::Wq, -1, {nq, W}), m.heads));
				proj.parts.push_back(by_map(tensor(i, TensorRole::Wk, -1, {nk, W}), m.kv_heads));
				proj.parts.push_back(mat(tensor(i, TensorRole::Wv, -1, {nv, W})));
				if (m.head_gate) proj.parts.push_back(mat(tensor(i, TensorRole::OutGate, -1, {m.heads, W})));
				if (m.qk_norm == yalm::QkNorm::PerHead) {
					pl.push_back({(void **)&L->qnorm, {vec32(tensor(i, TensorRole::QNorm, -1, {m.dim}))}});
					pl.push_back({(void **)&L->knorm, {vec32(tensor(i, TensorRole::KNorm, -1, {m.dim}))}});
				}
				{ // lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff, one number for the layer, in fp32 as the rest of the combination
					const float *v[4];
					const TensorRole roles[4] = {TensorRole::DiffLq1, TensorRole::DiffLk1, TensorRole::DiffLq2, TensorRole::DiffLk2};
					for (int k = 0; k < 4; ++k) v[k] = static_cast<const float *>(vec32(tensor(i, roles[k], -1, {m.dim})).first);
					float d1 = 0.f, d2 = 0.f;
					for (int d = 0; d < m.dim; ++d) d1 += v[0][d] * v[1][d], d2 += v[2][d] * v[3][d];
					L->lambda = expf(d1) - expf(d2) + m.diff;
				}
				pl.push_back({&L->wo, {mat(tensor(i, TensorRole::Wo, -1, {W, no}))}});
				if (m.rot.dims > 0) {
					std::vector<float> fr;
					m.rot.table(&fr, &L->rot_mag);
					_host_converted.emplace_back(fr.size() * sizeof(float));
					memcpy(_host_converted.back().data(), fr.data(), fr.size() * sizeof(float));
					pl.push_back({(void **)&L->rot_freq, {{_host_converted.back().data(), fr.size() * sizeof(float)}}});
				}
				// rings for the window, fp32 buffers for the kept first tokens (read like pooled blocks of one token)
				L->ring = m.window > 0 ? std::min(c.max_seq_len, (m.window + c.stack_chunk + 63) / 64 * 64) : c.max_seq_len;
				const size_t cb = c.weight_dtype == DType::F32 ? 4 : 2;
				L->state_allocs.push_back({&L->kring, (size_t)m.maps * m.kv_heads * L->ring * m.dim * cb});
				L->state_allocs.push_back({&L->vring, (size_t)m.kv_heads * L->ring * m.vdim * cb});
				L->max_blocks = m.window > 0 ? m.keep_first : 0;
				if (L->max_blocks > 0) {
					L->state_allocs.push_back({(void **)&L->kpool, (size_t)m.maps * m.kv_heads * L->max_blocks * m.dim * 4});
					L->state_allocs.push_back({(void **)&L->vpool, (size_t)m.kv_heads * L->max_blocks * m.vdim * 4});
				}
				if (m.dim > 512 || m.vdim > 512) die("differential attention: head sizes above 512 are not built");
			} else
				die("layers with a norm on both sides take latent attention or differential attention");
			pl.push_back(proj);
			if (f.kind == FfnSpec::Dense) {
				pl.push_back({(void **)&L->norm2, {vec32(tensor(i, TensorRole::Norm2, -1, {W}))}});
				pl.push_back({(void **)&L->norm2b, {vec32(tensor(i, TensorRole::Norm2Post, -1, {W}))}});
				if (f.gated) pl.push_back({&L->wgu, {mat(tensor(i, TensorRole::Gate, -1, {f.ff, W})), mat(tensor(i, TensorRole::Up, -1, {f.ff, W}))}});
				else pl.push_back({&L->wgu, {mat(tensor(i, TensorRole::Up, -1, {f.ff, W}))}});
				pl.push_back({&L->wdown, {mat(tensor(i, TensorRole::Down, -1, {W, f.ff}))}});
			} else if (f.kind != FfnSpec::None)
				die("layers with a norm on both sides take a dense feed-forward or none");
			if (s.token_side > 0) {
				pl.push_back({&L->side_gate, {mat(tensor(i, TensorRole::SideGate, -1, {s.token_side, W}))}});
				pl.push_back({&L->side_proj, {mat(tensor(i, TensorRole::SideProj, -1, {W, s.token_side}))}});
				pl.push_back({(void **)&L->side_norm, {vec32(tensor(i, TensorRole::SideNorm, -1, {W}))}});
			}
			_stack.push_back(L);
			continue;
		}
		if (L->spec.kind == yalm::MixerKind::LatentAttention || L->spec.kind == yalm::MixerKind::LinearAttention) {
			// ---- pre-norm layer: norm + input convolution per sublayer, one packed projection of the mixer's input, weighted sum over depth ----
			const int W = s.width, taps = s.input_conv;
			const yalm::LayerSpec &ls = L->spec;
			const FfnSpec &f = ls.ffn;
			pl.push_back({(void **)&L->norm1, {vec32(tensor(i, TensorRole::Norm1, -1, {W}))}});
			if (taps > 0) {
				pl.push_back({(void **)&L->inconv1, {vec32(tensor(i, TensorRole::InConv1, -1, {W, taps}))}});
				if (taps > 1) L->state_allocs.push_back({(void **)&L->inconv1_state, (size_t)(taps - 1) * W * 4});
			}
			if (s.depth_average) pl.push_back({(void **)&L->depth_w, {vec32(tensor(i, TensorRole::DepthWeights, -1, {i + 2}))}});
			Placement proj{&L->wproj, {}};
			if (ls.kind == yalm::MixerKind::LatentAttention) {
				load_latent(i, L, proj, W);
			} else {
				const yalm::GlaSpec &g = ls.gla;
				const int hd = g.heads * g.dim, hp = g.heads * g.vdim;
				L->o_q = 0, L->o_k = hd, L->o_v = 2 * hd, L->o_gate = 2 * hd + hp, L->o_a1 = 2 * hd + 2 * hp;
				proj.parts.push_back(mat(tensor(i, TensorRole::Wq, -1, {hd, W})));
				proj.parts.push_back(mat(tensor(i, TensorRole::Wk, -1, {hd, W})));
				proj.parts.push_back(mat(tensor(i, TensorRole::Wv, -1, {hp, W})));
				proj.parts.push_back(mat(tensor(i, TensorRole::OutGate, -1, {hp, W})));
				proj.parts.push_back(mat(tensor(i, TensorRole::GlaDecay1, -1, {g.decay_rank, W})));
				pl.push_back({&L->wa2, {mat(tensor(i, TensorRole::GlaDecay2, -1, {hd, g.decay_rank}))}});
				pl.push_back({(void **)&L->d_dt_bias, {vec32(tensor(i, TensorRole::GlaDecayBias, -1, {hd}))}});
				pl.push_back({(void **)&L->mix_norm, {vec32(tensor(i, TensorRole::GlaNorm, -1, {g.vdim}))}});
				pl.push_back({&L->wo, {mat(tensor(i, TensorRole::Wo, -1, {W, hp}))}});
				L->state_allocs.push_back({(void **)&L->scan_state, (size_t)g.heads * g.vdim * g.dim * 4});
				if (g.dim > 256) die("linear attention: key sizes above 256 are not built");
			}
			pl.push_back(proj);
			if (f.kind != FfnSpec::None) {
				pl.push_back({(void **)&L->norm2, {vec32(tensor(i, TensorRole::Norm2, -1, {W}))}});
				if (taps > 0) {
					pl.push_back({(void **)&L->inconv2, {vec32(tensor(i, TensorRole::InConv2, -1, {W, taps}))}});
					if (taps > 1) L->state_allocs.push_back({(void **)&L->inconv2_state, (size_t)(taps - 1) * W * 4});
				}
			}
			if (f.kind == FfnSpec::Dense) {
				pl.push_back({&L->wgu, {mat(tensor(i, TensorRole::Gate, -1, {f.ff, W})), mat(tensor(i, TensorRole::Up, -1, {f.ff, W}))}});
				pl.push_back({&L->wdown, {mat(tensor(i, TensorRole::Down, -1, {W, f.ff}))}});
			} else if (f.kind == FfnSpec::Moe) {
				if (f.experts > 0) {
					Placement g{&L->wg, {}}, u{&L->wu, {}}, d{&L->wdown, {}};
					for (int e = 0; e < f.experts; ++e) {
						g.parts.push_back(mat(tensor(i, TensorRole::Gate, e, {f.ff, W})));
						u.parts.push_back(mat(tensor(i, TensorRole::Up, e, {f.ff, W})));
						d.parts.push_back(mat(tensor(i, TensorRole::Down, e, {W, f.ff})));
					}
					pl.push_back(g), pl.push_back(u), pl.push_back(d);
				}
				pl.push_back({&L->router, {mat(tensor(i, TensorRole::Router, -1, {f.experts + f.identity, W}))}});
				if (f.choice_bias) pl.push_back({(void **)&L->router_bias, {vec32(tensor(i, TensorRole::RouterBias, -1, {f.experts + f.identity}))}});
				if (f.shared_ff > 0) {
					pl.push_back({&L->wsgu, {mat(tensor(i, TensorRole::SharedGate, -1, {f.shared_ff, W})), mat(tensor(i, TensorRole::SharedUp, -1, {f.shared_ff, W}))}});
					pl.push_back({&L->wsdown, {mat(tensor(i, TensorRole::SharedDown, -1, {W, f.shared_ff}))}});
				}
			}
			_stack.push_back(L);
			continue;
		}
		const int nq = m.heads * m.dim, nk = m.kv_heads * m.dim, nv = m.kv_heads * m.vdim, no = m.heads * m.vdim, W = s.width;
		pl.push_back({&L->wqkv,
		              {mat(tensor(i, TensorRole::Wq, -1, {nq, W})), mat(tensor(i, TensorRole::Wk, -1, {nk, W})), mat(tensor(i, TensorRole::Wv, -1, {nv, W}))}});
		pl.push_back({&L->wo, {mat(tensor(i, TensorRole::Wo, -1, {W, no}))}});
		if (m.qk_norm == yalm::QkNorm::WholeProjection) {
			pl.push_back({(void **)&L->qnorm, {vec32(tensor(i, TensorRole::QNorm, -1, {nq}))}});
			pl.push_back({(void **)&L->knorm, {vec32(tensor(i, TensorRole::KNorm, -1, {nk}))}});
		}
		if (m.v_mix) {
			L->vmode = have_first ? 2 : 1;
			have_first = true;
			if (L->vmode == 2) pl.push_back({(void **)&L->vmix, {vec32(tensor(i, TensorRole::VMix, -1, {}))}});
		}
		pl.push_back({(void **)&L->norm1, {vec32(tensor(i, TensorRole::Norm1, -1, {W}))}});
		const FfnSpec &f = L->spec.ffn;
		if (f.kind != FfnSpec::None) pl.push_back({(void **)&L->norm2, {vec32(tensor(i, TensorRole::Norm2, -1, {W}))}});
		if (f.kind == FfnSpec::Dense) {
			pl.push_back({&L->wgu, {mat(tensor(i, TensorRole::Gate, -1, {f.ff, W})), mat(tensor(i, TensorRole::Up, -1, {f.ff, W}))}});
			pl.push_back({&L->wdown, {mat(tensor(i, TensorRole::Down, -1, {W, f.ff}))}});
		} else if (f.kind == FfnSpec::Moe) {
			Placement g{&L->wg, {}}, u{&L->wu, {}}, d{&L->wdown, {}};
			for (int e = 0; e < f.experts; ++e) {
				g.parts.push_back(mat(tensor(i, TensorRole::Gate, e, {f.ff, W})));
				u.parts.push_back(mat(tensor(i, TensorRole::Up, e, {f.ff, W})));
				d.parts.push_back(mat(tensor(i, TensorRole::Down, e, {W, f.ff})));
			}
			pl.push_back(g), pl.push_back(u), pl.push_back(d);
			pl.push_back({&L->router, {mat(tensor(i, TensorRole::Router, -1, {f.experts, W}))}});
		}
		// cache geometry
		const int span = std::max(m.window, m.pool);
		L->ring = m.window > 0 ? std::min(c.max_seq_len, (span + c.stack_chunk + 63) / 64 * 64) : c.max_seq_len;
		L->max_blocks = m.pool > 0 ? c.max_seq_len / m.pool + 1 : 0;
		_stack.push_back(L);
	}
	// v blending reads the first blending layer's values of the same rows: the shapes must agree
	int first_nv = -1;
	for (auto &L : _stack)
		if (L->vmode) {
			const int nv = L->spec.mix.kv_heads * L->spec.mix.vdim;
			if (first_nv < 0) first_nv = nv;
			else if (nv != first_nv) die("value blending needs the same number of value channels in every blending layer");
		}
}

// layers whose cache and state are all in state_allocs (no key / value ring pair of the generic attention)
static bool own_state(const StackLayer &L) {
	return L.sandwich || L.spec.kind == yalm::MixerKind::LatentAttention || L.spec.kind == yalm::MixerKind::LinearAttention;
}

void Model::cuda_stack(int device) {
	Config &c = *config;
	const StackSpec &s = *c.stack;
	c.tp_rank = 0, c.tp_size = 1;
	_device = Device::CUDA;
	set_cuda_device(device);
	using yalm::DeviceArena;
	const size_t cb = c.weight_dtype == DType::F32 ? 4 : 2; // cache element: fp32 in the 32-bit mode, bf16 otherwise
	size_t need = 0;
	for (const Placement &p : _scratch->placements) need += DeviceArena::padded(p.bytes());
	for (auto &L : _stack) {
		const yalm::MixerSpec &m = L->spec.mix;
		for (auto &sa : L->state_allocs) need += DeviceArena::padded(sa.second);
		if (s.parallel_block || own_state(*L)) continue;
		need += DeviceArena::padded((size_t)m.kv_heads * L->ring * m.dim * cb) + DeviceArena::padded((size_t)m.kv_heads * L->ring * m.vdim * cb);
		if (m.pool > 0)
			need += DeviceArena::padded((size_t)m.kv_heads * L->max_blocks * m.dim * 4) + DeviceArena::padded((size_t)m.kv_heads * L->max_blocks * m.vdim * 4);
	}
	_arena = std::make_shared<DeviceArena>();
	if (int rc = _arena->reserve(need)) die(std::string("device allocation failed: ") + cudaGetErrorString((cudaError_t)rc));
	yalm::Uploader up;
	for (const Placement &p : _scratch->placements) {
		char *dst = static_cast<char *>(_arena->take(p.bytes()));
		if (!dst) die("device arena exhausted (loader sizing bug)");
		*p.slot = dst;
		for (auto &part : p.parts) {
			if (up.put(dst, part.first, part.second, 0, part.second, 1)) die("upload failed");
			dst += part.second;
			_device_bytes += part.second;
		}
	}
	for (auto &L : _stack) {
		const yalm::MixerSpec &m = L->spec.mix;
		for (auto &sa : L->state_allocs) {
			if (!(*sa.first = _arena->take(sa.second))) die("device arena exhausted (sequence state)");
			up.zero(*sa.first, sa.second);
			_device_bytes += sa.second;
		}
		if (s.parallel_block || own_state(*L)) continue;
		const size_t kb = (size_t)m.kv_heads * L->ring * m.dim * cb, vb = (size_t)m.kv_heads * L->ring * m.vdim * cb;
		L->kring = _arena->take(kb), L->vring = _arena->take(vb);
		if (!L->kring || !L->vring) die("device arena exhausted (cache)");
		up.zero(L->kring, kb), up.zero(L->vring, vb);
		_device_bytes += kb + vb;
		if (m.pool > 0) {
			const size_t pk = (size_t)m.kv_heads * L->max_blocks * m.dim * 4, pv = (size_t)m.kv_heads * L->max_blocks * m.vdim * 4;
			L->kpool = static_cast<float *>(_arena->take(pk)), L->vpool = static_cast<float *>(_arena->take(pv));
			if (!L->kpool || !L->vpool) die("device arena exhausted (pooled cache)");
			up.zero(L->kpool, pk), up.zero(L->vpool, pv);
			_device_bytes += pk + pv;
		}
	}
	if (up.finish()) die("upload failed");
	_upload_pinned = up.pinned();
	_scratch->placements.clear();
	_host_converted.clear();
	_host_converted.shrink_to_fit();
	// per-pass scratch for stack_chunk rows
	StackScratch &S = *_scratch;
	S.cap = c.stack_chunk;
	const size_t cap = S.cap, W = s.width, top = std::max(1, s.max_top()), ff = std::max(1, s.max_ff());
	const size_t nqkv = std::max((size_t)s.max_q_dim() + s.max_kv_dim() + s.max_v_dim(), (size_t)s.max_proj());
	bool side_bufs = s.parallel_block; // buffers beside q | k | v: shifted / convolved inputs, second-stage products, per-mixer outputs
	for (auto &L : _stack) side_bufs = side_bufs || own_state(*L);
	for (auto &L : _stack) // a layer that reads another layer's cache rows
		if (L->kv_owner >= 0 && L->kv_owner < (int)_stack.size() && !L->kring) L->kring = _stack[L->kv_owner]->kring, L->ring = _stack[L->kv_owner]->ring;
	// latent attention, prompt portions in 16-bit: the window's latents as one operand, their keys and values per head as rings
	size_t lat16 = 0, latkv = 0, lat_ek = 0, lat_ev = 0;
	for (auto &L : _stack) {
		const yalm::LayerSpec &ls = L->spec;
		if (ls.kind != yalm::MixerKind::LatentAttention) continue;
		if (ls.mix.dim > 0 && !L->wuv) L->wuv = static_cast<char *>(L->wuk) + (size_t)ls.mix.heads * ls.mix.dim * ls.latent.kv_rank * dtype_size(c.weight_dtype);
		if (c.weight_dtype == DType::F32 || (ls.mix.window < 1 && !L->sandwich)) continue;
		// the rows a portion sees: the window before it and itself, or (no window) everything the ring holds
		const size_t rows = ls.mix.window > 0 ? std::min<size_t>(L->ring, (size_t)ls.mix.window + c.stack_chunk) : (size_t)L->ring, H = ls.mix.heads;
		lat16 = std::max(lat16, rows * ls.latent.kv_rank * 2), latkv = std::max(latkv, rows * H * (ls.mix.dim + ls.mix.vdim) * 4);
		lat_ek = std::max(lat_ek, H * L->ring * (ls.mix.dim + ls.latent.rot_dim) * 2), lat_ev = std::max(lat_ev, H * L->ring * ls.mix.vdim * 2);
	}
	const size_t pb = side_bufs ? 1 : 0, nconv = std::max(1, s.max_conv()), naux = std::max(1, s.max_aux()), no = std::max(1, s.max_o_dim());
	const size_t kmax = std::max({W, (size_t)s.max_o_dim(), ff});
	size_t shared_ff = 0;
	for (const LayerSpec &l : s.layers) shared_ff = std::max<size_t>(shared_ff, l.ffn.shared_ff);
	const bool moe = s.max_experts() > 0 && c.weight_dtype != DType::F32; // the grouped route needs 16-bit operands
	auto pad = [](size_t b) { return (b + 255) / 256 * 256; };
	struct Slot {
		void **p;
		size_t bytes;
	} slots[] = {{(void **)&S.x, 4 * cap * W},           {(void **)&S.qkv, 4 * cap * nqkv},      {(void **)&S.vfirst, 4 * cap * std::max<size_t>(1, s.max_v_dim())},
	             {(void **)&S.att, 4 * cap * std::max<size_t>(1, s.max_o_dim())},                   {(void **)&S.y, 4 * cap * top * W},
	             {(void **)&S.gu, 4 * cap * 2 * ff},     {(void **)&S.h, 4 * cap * top * ff},    {(void **)&S.wts, 4 * cap * top},
	             {(void **)&S.xn, 4 * cap * W},          {(void **)&S.logits, 4 * cap * (size_t)s.vocab}, {(void **)&S.probs, 4 * cap},
	             {(void **)&S.a16, 2 * cap * top * kmax}, {(void **)&S.a16e, pb * 2 * cap * top * kmax}, {(void **)&S.a16r, pb * 2 * cap * top * kmax}, {(void **)&S.ids, 4 * cap * top},       {(void **)&S.tokens, 4 * cap},
	             {(void **)&S.want, 4 * cap},            {(void **)&S.targets, 4 * cap},
	             {(void **)&S.attn_ws, 4 * yalm_attn_window_pool_workspace(512)}, {(void **)&S.ticket, 256},
	             {(void **)&S.hs, pb * 4 * cap * W}, {(void **)&S.conv, pb * 4 * cap * nconv}, {(void **)&S.aux, pb * 4 * cap * naux},
	             {(void **)&S.scan, pb * 4 * cap * no}, {(void **)&S.att2, pb * 4 * cap * no}, {(void **)&S.y1, pb * 4 * cap * W}, {(void **)&S.y2, pb * 4 * cap * W},
	             {(void **)&S.hist, 4 * cap * W * (size_t)S.hist_slabs}, {(void **)&S.hsh, 4 * cap * shared_ff},
	             {(void **)&S.lat16, lat16}, {(void **)&S.latkv, latkv}, {(void **)&S.lat_ek, lat_ek}, {(void **)&S.lat_ev, lat_ev},
	             {(void **)&S.moe_gu, moe ? 4 * cap * top * 2 * ff : 0}, {(void **)&S.moe_ys, moe ? 4 * cap * top * W : 0}, {(void **)&S.order, 4 * cap * top}};
	size_t total = 0;
	for (auto &sl : slots) total += pad(sl.bytes);
	if (cudaMalloc((void **)&S.arena, total) != cudaSuccess) die("device allocation failed (pass scratch)");
	cudaMemset(S.arena, 0, total);
	char *p = S.arena;
	for (auto &sl : slots) *sl.p = sl.bytes ? p : nullptr, p += pad(sl.bytes);
	if (side_bufs)
		for (int i = 0; i < 2; ++i)
			if (cudaStreamCreateWithFlags(&S.side[i], cudaStreamNonBlocking) != cudaSuccess ||
			    cudaEventCreateWithFlags(&S.fork[i], cudaEventDisableTiming) != cudaSuccess ||
			    cudaEventCreateWithFlags(&S.join[i], cudaEventDisableTiming) != cudaSuccess)
				die("stream / event creation failed");
	if (cudaDeviceSynchronize() != cudaSuccess) die("device error after upload");
}

// ------------------------------------------------------------------------------------------------------------------------
// One pass: n rows whose tokens are in scratch.tokens (or in the control block), positions pos0 .. (or ctl)
// ------------------------------------------------------------------------------------------------------------------------
// y = alpha * x W^T.  16-bit weights and enough rows: activations rounded once to the weight type, product on the tcgen05
// tensor cores (prefill_gemm.cu); otherwise (fp32 mode, few rows, rows that are not 16-byte multiples) the SIMT routes,
// which keep the activations in fp32.
static int stack_linear(Model &, const Config &c, void *a16, float *y, int ldy, const float *x, int ldx, const void *w, int M, int N, int K,
                        float alpha, cudaStream_t st) {
	const int dt = static_cast<int>(c.weight_dtype);
	static const bool tc_off = [] { const char *e = getenv("YALM_STACK_TC"); return e && e[0] == '0'; }();
	if (!tc_off && dt != YALM_F32 && M >= 32 && K % 8 == 0 && K >= 8 && ldy % 4 == 0 && ((uintptr_t)y & 15) == 0 && ((uintptr_t)w & 15) == 0) {
		ST_TRY(yalm_cast_rows16(a16, x, ldx, M, K, dt == YALM_BF16, st));
		return yalm_gemm_16(y, ldy, a16, w, M, N, K, 0, dt == YALM_BF16, alpha, st);
	}
	// one row: the streaming GEMV of the .yalm decode path (x staged in shared memory, 16 weight loads in flight per lane)
	if (M == 1 && K % 8 == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)x & 15) == 0) return yalm_gemv_scaled(y, x, w, K, N, dt, alpha, st);
	return yalm_linear_rows(y, ldy, x, ldx, w, dt, M, N, K, alpha, st);
}

// One row, 16-bit or fp32 weights with 16-byte rows: the product and what follows it run as one launch (ops_stack_gemv.cu).
// YALM_STACK_FUSE=0: A/B against the separate kernels.
static bool gemv_fusable(const Config &c, int n, int K, const void *w, const void *x) {
	static const bool off = [] { const char *e = getenv("YALM_STACK_FUSE"); return e && e[0] == '0'; }();
	return !off && n == 1 && K % 8 == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)x & 15) == 0 && (size_t)K * dtype_size(c.weight_dtype) % 16 == 0;
}

// YALM_STACK_FUSE_BLOCK=1: a parallel block's decode row runs norm + token shift inside its projection's launch and the
// residual add as the tail of its last product.  Off by default: on B200 both measure 2 - 4 % slower per token than the two
// small launches they save (every CTA of the projection recomputes the row's mean square, and the last-CTA ticket costs a
// device-scope fence), inside the captured decode step.
static bool block_fuse_on() {
	const char *e = getenv("YALM_STACK_FUSE_BLOCK");
	return e && e[0] == '1';
}

// YALM_STACK_BRANCHES=0: a parallel block's decode row runs its sublayers one after the other on the caller's stream
static bool branches_off() { // read per call (a captured step keeps the shape it was captured with): tests compare both
	const char *e = getenv("YALM_STACK_BRANCHES");
	return e && e[0] == '0';
}

static bool attn_mma_off() { // YALM_STACK_ATTN_MMA=0: A/B against the SIMT kernel
	static const bool off = [] { const char *e = getenv("YALM_STACK_ATTN_MMA"); return e && e[0] == '0'; }();
	return off;
}

// Experts of a prompt portion on the tensor cores: the (row, expert) slots are sorted by expert on the host (one small copy
// of the chosen ids), each expert's rows are gathered into one 16-bit operand (scaled by the slot's weight when the weight
// multiplies the expert's input), and gate, up and down run as one tcgen05 product per expert that has rows; the down
// outputs go back to slot order, where the output norm sums a row's slots.  Same arithmetic as the slot kernels up to the
// rounding of the operands.
static bool moe_grouped_off() { // YALM_STACK_MOE_TC=0: A/B against the slot kernels
	static const bool off = [] { const char *e = getenv("YALM_STACK_MOE_TC"); return e && e[0] == '0'; }();
	return off;
}

int Model::stack_moe_grouped(StackScratch &S, const yalm::StackLayer &L, const float *x, void *a16, int n, int act, cudaStream_t st) {
	const Config &c = *config;
	const FfnSpec &f = L.spec.ffn;
	const int W = c.stack->width, ff = f.ff, top = f.top, E = f.experts, EA = f.experts + f.identity, ns = n * top, bf16 = c.weight_dtype == DType::BF16;
	std::vector<int> ids(ns), order(ns), start(EA + 1, 0); // identity experts sort behind the real ones and take no product
	ST_TRY(cudaMemcpyAsync(ids.data(), S.ids, sizeof(int) * ns, cudaMemcpyDeviceToHost, st));
	ST_TRY(cudaStreamSynchronize(st));
	for (int s = 0; s < ns; ++s) {
		if (ids[s] < 0 || ids[s] >= EA) return YALM_EINVAL;
		++start[ids[s] + 1];
	}
	for (int e = 0; e < EA; ++e) start[e + 1] += start[e];
	const int nr = start[E]; // slots of real experts
	{
		std::vector<int> at(start.begin(), start.end() - 1);
		for (int s = 0; s < ns; ++s) order[at[ids[s]]++] = s; // stable: slots of an expert stay in row order
	}
	ST_TRY(cudaMemcpyAsync(S.order, order.data(), sizeof(int) * ns, cudaMemcpyHostToDevice, st));
	if (f.identity > 0) ST_TRY(yalm_moe_identity_slots(S.y, W, x, W, S.ids, S.wts, n, top, W, E, f.weight_on_input ? 0 : 1, st));
	if (nr == 0) return (int)cudaGetLastError();
	ST_TRY(yalm_moe_gather_rows16(a16, x, W, S.order, S.wts, nr, top, W, bf16, f.weight_on_input ? 1 : 0, st));
	const size_t es = dtype_size(c.weight_dtype);
	for (int e = 0; e < E; ++e) {
		const int m = start[e + 1] - start[e];
		if (!m) continue;
		const char *a = static_cast<const char *>(a16) + (size_t)start[e] * W * 2;
		float *gu = S.moe_gu + (size_t)start[e] * 2 * ff;
		ST_TRY(yalm_gemm_16(gu, 2 * ff, a, static_cast<const char *>(L.wg) + (size_t)e * ff * W * es, m, ff, W, 0, bf16, 1.f, st));
		ST_TRY(yalm_gemm_16(gu + ff, 2 * ff, a, static_cast<const char *>(L.wu) + (size_t)e * ff * W * es, m, ff, W, 0, bf16, 1.f, st));
	}
	ST_TRY(yalm_glu_act_rows(S.h, S.moe_gu, nr, ff, act, f.act_alpha, f.limit, f.up_offset, st));
	ST_TRY(yalm_cast_rows16(a16, S.h, ff, nr, ff, bf16, st));
	for (int e = 0; e < E; ++e) {
		const int m = start[e + 1] - start[e];
		if (!m) continue;
		ST_TRY(yalm_gemm_16(S.moe_ys + (size_t)start[e] * W, W, static_cast<const char *>(a16) + (size_t)start[e] * ff * 2,
		                    static_cast<const char *>(L.wdown) + (size_t)e * W * ff * es, m, W, ff, 0, bf16, 1.f, st));
	}
	ST_TRY(yalm_moe_scatter_rows(S.y, W, S.moe_ys, W, S.order, S.wts, nr, W, f.weight_on_input ? 0 : 1, st));
	return (int)cudaGetLastError(); // `order` was pageable host memory: the copy call returned after staging it
}

// One parallel block over n rows: h = norm(x); the mixer reads the token-shifted h through ONE packed projection, the experts
// read h itself; x += mixer + experts.  What the rows leave for the next call (previous h, convolution tails, matrix states,
// keys) is written by the ops themselves.
int Model::stack_layer_parallel(StackScratch &S, const yalm::StackLayer &L, int n, int pos0, const int *ctl, cudaStream_t st) {
	const Config &c = *config;
	const StackSpec &sp = *c.stack;
	const yalm::LayerSpec &ls = L.spec;
	const int dt = static_cast<int>(c.weight_dtype), W = sp.width, f32 = c.weight_dtype == DType::F32;
	const float woff = sp.norm_one_plus ? 1.f : 0.f;
	const int ldp = ls.proj_width();
	float *P = S.qkv;
	const bool fuse = n == 1 && block_fuse_on();
	const bool branch = !fuse && !branches_off(); // independent sublayers on side streams, see below
	cudaStream_t se = st, sr = st;                // the experts' and the delta rule's streams
	const FfnSpec &f = ls.ffn;
	const int nsum = f.kind == FfnSpec::Moe ? f.top : 0;
	// The experts only need h.  A prompt portion forks them before the projection (its product leaves SMs idle at small widths:
	// +7 % at width 1024); a decode row forks them after it: the projection streams its weights at the memory's rate, the mixer's
	// small kernels after it do not, and that is where the experts' traffic fits (forking earlier measured 5 % slower per row).
	auto fork_experts = [&]() -> int {
		if (branch && nsum) {
			se = S.side[0];
			ST_TRY(cudaEventRecord(S.fork[0], st));
			ST_TRY(cudaStreamWaitEvent(se, S.fork[0], 0));
		}
		return 0;
	};
	if (fuse && sp.token_shift && gemv_fusable(c, n, W, L.wproj, S.x)) // a decode row: norm, shift and projection as one launch
		ST_TRY(yalm_gemv_norm_shift(P, S.x, L.wproj, W, ldp, dt, L.norm1, sp.norm_scalar, woff, sp.norm_eps, L.shift, L.hprev, S.xn, pos0, ctl, S.ticket, st));
	else {
		ST_TRY(yalm_norm_shift_rows(S.xn, sp.token_shift ? S.hs : nullptr, S.x, L.norm1, sp.norm_scalar, woff, sp.norm_eps, L.shift, L.hprev, n, W, pos0, ctl, st));
		if (n > 1) ST_TRY(fork_experts());
		ST_TRY(stack_linear(*this, c, S.a16, P, ldp, sp.token_shift ? S.hs : S.xn, W, L.wproj, n, ldp, W, 1.f, st));
	}
	if (n == 1) ST_TRY(fork_experts());
	// The experts (which read h), the attention and the delta rule (which read disjoint columns of the projection and own their
	// scratch and 16-bit operand buffers) are independent: they run on side streams forked here and joined before the residual
	// add.  A decode row is a chain of small launches, a prompt portion's products leave most SMs idle (16 to 64 CTAs each): both
	// overlap.  Inside a captured decode step the streams become parallel branches of the graph.
	// ---- experts on h ----
	auto experts = [&]() -> int {
		if (!nsum) return 0;
		const int act = f.act == yalm::GluAct::SigmoidScaled ? 2 : f.act == yalm::GluAct::Silu ? YALM_ACT_SILU : YALM_ACT_GELU;
		ST_TRY(yalm_router_topk_rows(S.ids, S.wts, S.xn, W, L.router, dt, n, f.experts, f.top, W, f.score == yalm::RouterScore::Sigmoid ? 1 : 0,
		                             f.renormalize ? 1 : 0, f.renorm_eps, f.groups, f.keep_groups, se));
		if (S.moe_gu && !ctl && n * f.top >= 64 && W % 8 == 0 && f.ff % 8 == 0 && !moe_grouped_off())
			return stack_moe_grouped(S, L, S.xn, se == st ? S.a16 : S.a16e, n, act, se); // waits on the host for the chosen experts
		ST_TRY(yalm_moe_glu_slots(S.h, S.xn, W, L.wg, L.wu, dt, S.ids, S.wts, n, f.top, f.ff, W, act, f.act_alpha, f.limit, f.up_offset,
		                          f.weight_on_input ? 1 : 0, se));
		return yalm_moe_down_slots(S.y, W, S.h, L.wdown, dt, S.ids, S.wts, n, f.top, f.ff, W, f.weight_on_input ? 0 : 1, se);
	};
	if (!branch) ST_TRY(experts()); // one stream: before the mixer, whose last product can then carry the block's residual add
	auto join = [&]() -> int { // the side streams' work precedes what follows on the caller's stream
		if (se != st) {
			ST_TRY(cudaEventRecord(S.join[0], se));
			ST_TRY(cudaStreamWaitEvent(st, S.join[0], 0));
		}
		if (sr != st) {
			ST_TRY(cudaEventRecord(S.join[1], sr));
			ST_TRY(cudaStreamWaitEvent(st, S.join[1], 0));
		}
		return 0;
	};
	const float *mix_b = nullptr;
	if (ls.kind == yalm::MixerKind::StateSpace) {
		const yalm::SsmSpec &q = ls.ssm;
		const int inner = q.inner(), C = q.conv_channels(), gn = q.groups * q.state, o_dt = 2 * inner + 2 * gn;
		ST_TRY(yalm_conv_act_rows(S.conv, C, P + inner, ldp, L.conv_w, L.conv_b, L.conv_state, n, C, q.conv, pos0, ctl, st));
		ST_TRY(yalm_ssm_prep_rows(P + o_dt, ldp, S.aux, q.heads, L.dt_bias, L.a_log, n, q.heads, st));
		ST_TRY(yalm_state_scan_rows(S.scan, inner, S.conv + inner, C, S.conv + inner + gn, C, S.conv, C, S.aux, q.heads, 0, P + o_dt, ldp, nullptr, 0, L.skip,
		                            L.scan_state, n, q.heads, q.heads / q.groups, q.state, q.vdim, pos0, ctl, st));
		ST_TRY(yalm_gated_group_norm_rows(S.att, inner, S.scan, inner, P, ldp, L.mix_norm, n, inner, q.norm_groups, sp.norm_eps, st));
		if (fuse && gemv_fusable(c, n, inner, L.wout, S.att)) return yalm_gemv_residual_sum(S.x, S.y1, S.att, L.wout, 1.f, inner, W, dt, nullptr, S.y, nsum, W, S.ticket, st);
		ST_TRY(stack_linear(*this, c, S.a16, S.y1, W, S.att, inner, L.wout, n, W, inner, 1.f, st));
	} else {
		if (branch) {
			sr = S.side[1];
			ST_TRY(cudaEventRecord(S.fork[1], st));
			ST_TRY(cudaStreamWaitEvent(sr, S.fork[1], 0));
		}
		// ---- left: sigmoid attention over the key ring and the kept first tokens ----
		const yalm::MixerSpec &m = ls.mix;
		const int nq = m.heads * m.dim, no = m.heads * m.vdim;
		const int keep = m.window > 0 ? m.keep_first : 0;
		ST_TRY(yalm_qk_bias_append_rows(P + L.o_q, P + L.o_k, ldp, L.qkb, L.qkb + nq, L.kring, L.kfirst, n, m.heads, m.kv_heads, m.dim, L.ring, keep, f32, pos0,
		                                ctl, st));
		// many rows over the bf16 ring: tensor cores; decode-sized calls, the fp32 ring and other head sizes: the SIMT kernel
		if (!f32 && n >= 16 && ldp % 4 == 0 && L.o_q % 4 == 0 && L.o_gate % 2 == 0 && no % 2 == 0 && yalm_attn_sigmoid_mma_shape(m.dim) && !attn_mma_off())
			ST_TRY(yalm_attn_sigmoid_mma(S.att, no, P + L.o_q, ldp, L.kring, L.kfirst, P + L.o_gate, ldp, L.rel, L.bucket, L.head_bias, L.bias_table, c.max_seq_len, n, m.heads,
			                             m.kv_heads, m.dim, L.ring, m.window, keep, m.scale, c.max_seq_len, pos0, ctl, st));
		else
			ST_TRY(yalm_attn_sigmoid_rows(S.att, no, P + L.o_q, ldp, L.kring, L.kfirst, P + L.o_gate, ldp, L.rel, L.bucket, L.head_bias, S.attn_ws, n, m.heads,
			                              m.kv_heads, m.dim, L.ring, m.window, keep, m.scale, f32, c.max_seq_len, pos0, ctl, st));
		ST_TRY(stack_linear(*this, c, S.a16, S.y1, W, S.att, no, L.wo, n, W, no, ls.left_scale, st));
		// ---- right: gated delta rule ----
		const yalm::DeltaSpec &d = ls.delta;
		const int dk = d.kv_heads * d.dim, dv = d.heads * d.vdim, dg = d.heads * d.dim, C = 2 * dk + dv, lda = dg + dv;
		ST_TRY(yalm_conv_act_rows(S.conv, C, P + L.o_dq, ldp, L.conv_w, nullptr, L.conv_state, n, C, d.conv, pos0, ctl, sr));
		ST_TRY(stack_linear(*this, c, sr == st ? S.a16 : S.a16r, S.aux, lda, P + L.o_a1, ldp, L.wa2, n, dg, d.decay_rank, 1.f, sr));
		ST_TRY(stack_linear(*this, c, sr == st ? S.a16 : S.a16r, S.aux + dg, lda, P + L.o_g1, ldp, L.wg2, n, dv, d.gate_rank, 1.f, sr));
		ST_TRY(yalm_delta_prep_rows(S.conv, S.conv + dk, C, P + L.o_beta, ldp, S.aux, lda, L.d_a_log, L.d_dt_bias, n, d.heads, d.kv_heads, d.dim, 1e-6f,
		                            1.0f / sqrtf((float)d.dim), sr));
		ST_TRY(yalm_state_scan_rows(S.scan, dv, S.conv + dk, C, S.conv, C, S.conv + 2 * dk, C, S.aux, lda, 1, nullptr, 0, P + L.o_beta, ldp, nullptr,
		                            L.scan_state, n, d.heads, d.heads / d.kv_heads, d.dim, d.vdim, pos0, ctl, sr));
		ST_TRY(yalm_head_norm_gate_rows(S.att2, dv, S.scan, dv, S.aux + dg, lda, L.d_norm, n, d.heads, d.vdim, sp.norm_eps, sr));
		if (fuse && gemv_fusable(c, n, dv, L.wout, S.att2)) return yalm_gemv_residual_sum(S.x, S.y2, S.att2, L.wout, ls.right_scale, dv, W, dt, S.y1, S.y, nsum, W, S.ticket, st);
		ST_TRY(stack_linear(*this, c, sr == st ? S.a16 : S.a16r, S.y2, W, S.att2, dv, L.wout, n, W, dv, ls.right_scale, sr));
		mix_b = S.y2;
	}
	if (branch) ST_TRY(experts()); // enqueued last: its host wait (prompt portions) then overlaps the mixer's kernels
	ST_TRY(join());
	return yalm_residual_sum_rows(S.x, S.y1, mix_b, S.y, W, nsum, n, W, st);
}

static int glu_act_code(yalm::GluAct a) {
	return a == yalm::GluAct::SigmoidScaled ? 2 : a == yalm::GluAct::GeluTanh ? 3 : a == yalm::GluAct::Silu ? YALM_ACT_SILU : YALM_ACT_GELU;
}

// One pre-norm layer over n rows: u = N1(x) + conv(N1(x)), x += mixer(u); v = N2(x) + conv(N2(x)), x += ff(v); then the
// layer's result joins the earlier ones and x becomes their weighted sum.  The mixer is latent attention over cached rows
// [latent | rotated key part] (its own, or another layer's) or gated linear attention over a matrix state.  What the rows
// leave for the next call (normed inputs of both convolutions, cache rows, matrix state) is written by the ops themselves.
int Model::stack_layer_prenorm(StackScratch &S, const yalm::StackLayer &L, int index, int n, int pos0, const int *ctl, cudaStream_t st) {
	const Config &c = *config;
	const StackSpec &sp = *c.stack;
	const yalm::LayerSpec &ls = L.spec;
	const int dt = static_cast<int>(c.weight_dtype), W = sp.width, f32 = c.weight_dtype == DType::F32, taps = std::max(1, sp.input_conv);
	const int ldp = ls.proj_width();
	float *P = S.qkv;
	// ---- token mixer ----
	ST_TRY(yalm_norm_conv_rows(S.hs, S.xn, S.x, L.norm1, sp.layer_norm ? 1 : 0, sp.norm_eps, L.inconv1, L.inconv1_state, n, W, taps, pos0, ctl, st));
	ST_TRY(stack_linear(*this, c, S.a16, P, ldp, S.hs, W, L.wproj, n, ldp, W, 1.f, st));
	if (ls.kind == yalm::MixerKind::LatentAttention) {
		const yalm::MixerSpec &m = ls.mix;
		const yalm::LatentSpec &a = ls.latent;
		const int row = a.kv_rank + a.rot_dim, nq = m.heads * (m.dim + a.rot_dim), nqa = m.heads * row, nl = m.heads * a.kv_rank, no = m.heads * m.vdim;
		const bool own = a.kv_from < 0;
		ST_TRY(yalm_latent_post_rows(P, ldp, L.o_q, a.q_rank, L.qnorm, L.o_kv, a.kv_rank, a.rot_dim, L.knorm, own ? L.kring : nullptr, L.ring, L.rot_freq,
		                             L.rot_mag, a.rot.dims, a.rot.interleaved ? 1 : 0, sp.norm_eps, f32, n, pos0, ctl, st));
		ST_TRY(stack_linear(*this, c, S.a16, S.conv, nq, P + L.o_q, ldp, L.wuq, n, nq, a.q_rank, 1.f, st));
		const int dk = m.dim + a.rot_dim;
		if (!f32 && !ctl && n >= 16 && m.window > 0 && m.dim > 0 && S.lat16 && a.kv_rank % 8 == 0 && nq % 4 == 0 && no % 2 == 0 && (m.heads * (m.dim + m.vdim)) % 4 == 0 &&
		    yalm_attn_window_pool_mma_shape(dk, m.vdim) && !attn_mma_off()) {
			// A prompt portion in 16-bit: the latents of the visible rows times [W_uk ; W_uv] on the tensor cores give every head's keys
			// and values, written beside the rotated key part into head-major rings for the windowed tensor-core attention; the queries
			// stay as projected, their rotated part turned in place.
			const int first = std::max(0, pos0 - m.window + 1), count = pos0 + n - first, nkv = m.heads * (m.dim + m.vdim);
			ST_TRY(yalm_latent_gather_rows16(S.lat16, L.kring, L.ring, row, a.kv_rank, first, count, st));
			ST_TRY(yalm_gemm_16(S.latkv, nkv, S.lat16, L.wuk, count, nkv, a.kv_rank, 0, dt == YALM_BF16, 1.f, st));
			ST_TRY(yalm_latent_pack_rings(S.lat_ek, S.lat_ev, S.latkv, nkv, L.kring, L.ring, a.kv_rank, a.rot_dim, m.heads, m.dim, m.vdim, L.ring, first, count, st));
			ST_TRY(yalm_rotate_heads_rows(S.conv, nq, m.heads, dk, m.dim, L.rot_freq, L.rot_mag, a.rot.dims, a.rot.interleaved ? 1 : 0, n, pos0, ctl, st));
			ST_TRY(yalm_attn_window_pool_mma(S.att, no, S.conv, nq, S.lat_ek, S.lat_ev, nullptr, nullptr, n, m.heads, m.heads, dk, m.vdim, L.ring, 0, m.window, 0,
			                                 m.scale, pos0, ctl, st));
			if (m.out_gate) ST_TRY(yalm_sigmoid_gate_rows(S.att, no, P + L.o_gate, ldp, n, no, st));
		} else {
			// A decode row (and what the tensor-core route does not take): W_uk moves to the query side, every head reads the one cached
			// row of a position — keys are whole rows, values their first kv_rank channels — and W_uv follows the weighted sum.
			ST_TRY(yalm_latent_query_rows(S.aux, nqa, S.conv, nq, L.wukt, dt, n, m.heads, m.dim, a.rot_dim, a.kv_rank, L.rot_freq, L.rot_mag, a.rot.dims,
			                              a.rot.interleaved ? 1 : 0, pos0, ctl, st));
			static const bool one_pass_off = [] { const char *e = getenv("YALM_STACK_ATTN_LANES"); return e && e[0] == '0'; }();
			if (!f32 && !one_pass_off && yalm_attn_latent_rows_shape(row, a.kv_rank, row) && ((uintptr_t)L.kring & 15) == 0 && nqa % 4 == 0)
				ST_TRY(yalm_attn_latent_rows(S.scan, nl, S.aux, nqa, L.kring, row, S.attn_ws, n, m.heads, row, a.kv_rank, L.ring, m.window, m.scale, c.max_seq_len,
				                             pos0, ctl, st));
			else
				ST_TRY(yalm_attn_window_pool_strided(S.scan, nl, S.aux, nqa, L.kring, row, L.kring, row, nullptr, nullptr, S.attn_ws, n, m.heads, 1, row, a.kv_rank,
				                                     L.ring, 0, m.window, 0, m.scale, f32, c.max_seq_len, pos0, ctl, st));
			ST_TRY(yalm_head_linear_gate_rows(S.att, no, S.scan, nl, L.wuv, dt, m.out_gate ? P + L.o_gate : nullptr, ldp, n, m.heads, m.vdim, a.kv_rank, st));
		}
		ST_TRY(stack_linear(*this, c, S.a16, S.y1, W, S.att, no, L.wo, n, W, no, 1.f, st));
	} else {
		const yalm::GlaSpec &g = ls.gla;
		const int hd = g.heads * g.dim, hp = g.heads * g.vdim;
		ST_TRY(stack_linear(*this, c, S.a16, S.aux, hd, P + L.o_a1, ldp, L.wa2, n, hd, g.decay_rank, 1.f, st));
		ST_TRY(yalm_gla_prep_rows(S.aux, hd, L.d_dt_bias, g.tau, P + L.o_q, ldp, 1.0f / sqrtf((float)g.dim), n, hd, st));
		ST_TRY(yalm_state_scan_rows(S.scan, hp, P + L.o_k, ldp, P + L.o_q, ldp, P + L.o_v, ldp, S.aux, hd, 1, nullptr, 0, nullptr, 0, nullptr, L.scan_state, n,
		                            g.heads, 1, g.dim, g.vdim, pos0, ctl, st));
		ST_TRY(yalm_head_norm_act_rows(S.att, hp, S.scan, hp, P + L.o_gate, ldp, L.mix_norm, n, g.heads, g.vdim, sp.norm_eps, 1, st));
		ST_TRY(stack_linear(*this, c, S.a16, S.y1, W, S.att, hp, L.wo, n, W, hp, 1.f, st));
	}
	// ---- feed-forward ----
	const FfnSpec &f = ls.ffn;
	const float *add_a = S.y1, *add_b = nullptr, *slots = nullptr;
	int nsum = 0;
	if (f.kind != FfnSpec::None) {
		ST_TRY(yalm_add_norm_conv_rows(S.hs, S.xn, S.x, S.y1, L.norm2, sp.layer_norm ? 1 : 0, sp.norm_eps, L.inconv2, L.inconv2_state, n, W, taps, pos0, ctl, st));
		add_a = nullptr;
		const int act = glu_act_code(f.act);
		if (f.kind == FfnSpec::Dense) {
			ST_TRY(stack_linear(*this, c, S.a16, S.gu, 2 * f.ff, S.hs, W, L.wgu, n, 2 * f.ff, W, 1.f, st));
			ST_TRY(yalm_glu_act_rows(S.h, S.gu, n, f.ff, act, f.act_alpha, f.limit, f.up_offset, st));
			ST_TRY(stack_linear(*this, c, S.a16, S.y1, W, S.h, f.ff, L.wdown, n, W, f.ff, 1.f, st));
			add_a = S.y1;
		} else {
			const int EA = f.experts + f.identity;
			cudaStream_t ss = st;
			if (f.shared_ff > 0) {
				// The shared expert and the routed ones both read the same input and own their buffers: the shared expert runs on a
				// side stream (a parallel branch of the captured decode step), enqueued first because the grouped route of a prompt
				// portion waits on the host for the chosen experts.
				if (!branches_off() && S.side[0]) {
					ss = S.side[0];
					ST_TRY(cudaEventRecord(S.fork[0], st));
					ST_TRY(cudaStreamWaitEvent(ss, S.fork[0], 0));
				}
				ST_TRY(stack_linear(*this, c, ss == st ? S.a16 : S.a16e, S.gu, 2 * f.shared_ff, S.hs, W, L.wsgu, n, 2 * f.shared_ff, W, 1.f, ss));
				ST_TRY(yalm_glu_act_rows(S.hsh, S.gu, n, f.shared_ff, glu_act_code(f.shared_act), 1.f, 0.f, 0.f, ss));
				ST_TRY(stack_linear(*this, c, ss == st ? S.a16 : S.a16e, S.y2, W, S.hsh, f.shared_ff, L.wsdown, n, W, f.shared_ff, 1.f, ss));
				add_b = S.y2;
			}
			ST_TRY(yalm_router_bias_topk_rows(S.ids, S.wts, S.hs, W, L.router, dt, n, EA, f.top, W, f.score == yalm::RouterScore::Sigmoid ? 1 : 0,
			                                  f.renormalize ? 1 : 0, f.renorm_eps, 1, 1, f.choice_bias ? L.router_bias : nullptr, f.router_scale, st));
			if (S.moe_gu && !ctl && f.experts > 0 && n * f.top >= 64 && W % 8 == 0 && f.ff % 8 == 0 && !moe_grouped_off())
				ST_TRY(stack_moe_grouped(S, L, S.hs, S.a16, n, act, st));
			else {
				if (f.experts > 0)
					ST_TRY(yalm_moe_glu_slots_real(S.h, S.hs, W, L.wg, L.wu, dt, S.ids, S.wts, n, f.top, f.ff, W, act, f.act_alpha, f.limit, f.up_offset,
					                               f.weight_on_input ? 1 : 0, f.experts, st));
				ST_TRY(yalm_moe_down_slots_real(S.y, W, S.h, L.wdown, dt, S.ids, S.wts, n, f.top, f.ff, W, f.weight_on_input ? 0 : 1, f.experts, S.hs, W, st));
			}
			slots = S.y, nsum = f.top;
			if (ss != st) {
				ST_TRY(cudaEventRecord(S.join[0], ss));
				ST_TRY(cudaStreamWaitEvent(st, S.join[0], 0));
			}
		}
	}
	// the layer's result (x + what is still to be added) joins the earlier ones; x becomes their weighted sum
	if (sp.depth_average)
		return yalm_depth_average_rows(S.x, S.hist, (size_t)S.cap * W, L.depth_w, index + 2, n, W, add_a, add_b, slots, W, nsum, st);
	return yalm_residual_sum_rows(S.x, add_a, add_b, slots, W, nsum, n, W, st);
}

static int plain_act_code(yalm::GluAct a) {
	return a == yalm::GluAct::GeluErf ? 4 : a == yalm::GluAct::GeluTanh ? 3 : a == yalm::GluAct::Silu ? YALM_ACT_SILU : YALM_ACT_GELU;
}

// One layer with a norm on both sides of each sublayer over n rows: x += N1b(mixer(N1(x))), x += N2b(ff(N2(x))), then the token
// side input.  The mixer is latent attention with full-rank queries and a sink per head over cached rows [latent | rotated key
// part] (its own, or another layer's), or differential attention: (map, head) is one list of attention heads over rings that
// hold (map, kv head) key vectors and kv heads values, the window's kept first tokens are read like pooled blocks of one token,
// and the two maps of a head are combined afterwards.  What the rows leave for the next call is written by the ops themselves.
static bool side_one_kernel() { // YALM_STACK_SIDE=0: the token side input as one launch of one CTA per row (the route of sizes that are no 16-byte multiples)
	static const bool on = [] { const char *e = getenv("YALM_STACK_SIDE"); return e && e[0] == '0'; }();
	return on;
}

int Model::stack_layer_sandwich(StackScratch &S, const yalm::StackLayer &L, const yalm::StackLayer *next, int index, int n, int pos0, const int *ctl,
                                bool from_ctl, cudaStream_t st) {
	const Config &c = *config;
	const StackSpec &sp = *c.stack;
	const yalm::LayerSpec &ls = L.spec;
	const yalm::MixerSpec &m = ls.mix;
	const int dt = static_cast<int>(c.weight_dtype), W = sp.width, f32 = c.weight_dtype == DType::F32;
	const int ldp = ls.proj_width(), no = m.heads * m.vdim;
	float *P = S.qkv;
	const FfnSpec &f = ls.ffn;
	const bool side = sp.token_side > 0;
	// A decode row's products end in a tail that has the finished residual row in one CTA: the next sublayer's input norm rides along
	// (xn_valid tells the next sublayer), so that only the first layer of a step launches a norm of its own.
	const float *norm_after_mixer = f.kind == FfnSpec::Dense ? L.norm2 : (side || !next) ? nullptr : next->norm1;
	const float *norm_after_ffn = (side || !next) ? nullptr : next->norm1;
	const float *norm_after_side = next ? next->norm1 : nullptr;
	// ---- token mixer ----
	if (!S.xn_valid) ST_TRY(yalm_norm_shift_rows(S.xn, nullptr, S.x, L.norm1, 0, 0.f, sp.norm_eps, nullptr, nullptr, n, W, pos0, ctl, st));
	S.xn_valid = false;
	if (ls.kind == yalm::MixerKind::LatentAttention) {
		const yalm::LatentSpec &a = ls.latent;
		const int row = a.kv_rank + a.rot_dim, nqa = m.heads * row, nl = m.heads * a.kv_rank, dk = m.dim + a.rot_dim;
		const bool own = a.kv_from < 0;
		ST_TRY(stack_linear(*this, c, S.a16, P, ldp, S.xn, W, L.wproj, n, ldp, W, 1.f, st));
		if (own)
			ST_TRY(yalm_latent_post_rows(P, ldp, L.o_q, 0, nullptr, L.o_kv, a.kv_rank, a.rot_dim, L.knorm, L.kring, L.ring, L.rot_freq, L.rot_mag, a.rot.dims,
			                             a.rot.interleaved ? 1 : 0, sp.norm_eps, f32, n, pos0, ctl, st));
		float *Q = P + L.o_q; // the queries as projected, per head [unrotated | rotated part]
		if (!f32 && !ctl && n >= 16 && m.dim > 0 && S.lat16 && a.kv_rank % 8 == 0 && ldp % 4 == 0 && no % 2 == 0 && (m.heads * (m.dim + m.vdim)) % 4 == 0 &&
		    yalm_attn_window_pool_mma_shape(dk, m.vdim) && !attn_mma_off()) {
			// A prompt portion in 16-bit: the latents of the visible rows times [W_uk ; W_uv] on the tensor cores give every head's keys
			// and values, written beside the rotated key part into head-major rings for the tensor-core attention.
			const int first = m.window > 0 ? std::max(0, pos0 - m.window + 1) : 0, count = pos0 + n - first, nkv = m.heads * (m.dim + m.vdim);
			ST_TRY(yalm_latent_gather_rows16(S.lat16, L.kring, L.ring, row, a.kv_rank, first, count, st));
			ST_TRY(yalm_gemm_16(S.latkv, nkv, S.lat16, L.wuk, count, nkv, a.kv_rank, 0, dt == YALM_BF16, 1.f, st));
			ST_TRY(yalm_latent_pack_rings(S.lat_ek, S.lat_ev, S.latkv, nkv, L.kring, L.ring, a.kv_rank, a.rot_dim, m.heads, m.dim, m.vdim, L.ring, first, count, st));
			ST_TRY(yalm_rotate_heads_rows(Q, ldp, m.heads, dk, m.dim, L.rot_freq, L.rot_mag, a.rot.dims, a.rot.interleaved ? 1 : 0, n, pos0, ctl, st));
			ST_TRY(yalm_attn_window_pool_mma_sink(S.att, no, Q, ldp, S.lat_ek, S.lat_ev, nullptr, nullptr, n, m.heads, m.heads, dk, m.vdim, L.ring, 0, m.window, 0,
			                                      m.scale, pos0, ctl, L.sink, m.heads, st));
		} else {
			// A decode row (and what the tensor-core route does not take): W_uk moves to the query side, every head reads the one cached
			// row of a position — keys are whole rows, values their first kv_rank channels — and W_uv follows the weighted sum.
			ST_TRY(yalm_latent_query_rows(S.aux, nqa, Q, ldp, L.wukt, dt, n, m.heads, m.dim, a.rot_dim, a.kv_rank, L.rot_freq, L.rot_mag, a.rot.dims,
			                              a.rot.interleaved ? 1 : 0, pos0, ctl, st));
			static const bool latent_mma_off = [] { const char *e = getenv("YALM_STACK_LATENT_MMA"); return e && e[0] == '0'; }(); // A/B against the SIMT kernel
			if (!f32 && !latent_mma_off && yalm_attn_latent_mma_shape(row, a.kv_rank, row) && ((uintptr_t)L.kring & 15) == 0 && nqa % 4 == 0 && n * m.heads <= 4096) {
				// the heads as the M tile of the tensor cores; the keys a row can ever see, in tiles of 64, are split over up to 128 CTAs (shapes only)
				const int tiles = ((m.window > 0 ? std::min(m.window, c.max_seq_len) : c.max_seq_len) + 63) / 64, ctas = (m.heads + 15) / 16 * n;
				const int cap = std::max(1, std::min({tiles, 128, 4096 / (n * m.heads), (296 + ctas - 1) / ctas}));
				const int per = (tiles + cap - 1) / cap, nsplit = (tiles + per - 1) / per;
				ST_TRY(yalm_attn_latent_mma_rows(S.scan, nl, S.aux, nqa, L.kring, row, S.attn_ws, n, m.heads, row, a.kv_rank, L.ring, m.window, m.scale, nsplit, pos0,
				                                 ctl, L.sink, st));
			} else if (!f32 && yalm_attn_latent_rows_shape(row, a.kv_rank, row) && ((uintptr_t)L.kring & 15) == 0 && nqa % 4 == 0)
				ST_TRY(yalm_attn_latent_rows_sink(S.scan, nl, S.aux, nqa, L.kring, row, S.attn_ws, n, m.heads, row, a.kv_rank, L.ring, m.window, m.scale,
				                                  c.max_seq_len, pos0, ctl, L.sink, st));
			else
				ST_TRY(yalm_attn_window_pool_sink(S.scan, nl, S.aux, nqa, L.kring, row, L.kring, row, nullptr, nullptr, S.attn_ws, n, m.heads, 1, row, a.kv_rank,
				                                  L.ring, 0, m.window, 0, m.scale, f32, c.max_seq_len, pos0, ctl, L.sink, 1, st));
			ST_TRY(yalm_head_linear_gate_rows(S.att, no, S.scan, nl, L.wuv, dt, nullptr, 0, n, m.heads, m.vdim, a.kv_rank, st));
		}
	} else {
		const int nqv = m.maps * m.heads, nkv = m.maps * m.kv_heads, ncols = L.o_gate + (m.head_gate ? m.heads : 0), na = m.maps * no;
		const int keep = L.max_blocks, pool = keep > 0 ? 1 : 0;
		ST_TRY(stack_linear(*this, c, S.a16, P, ldp, S.xn, W, L.wproj, n, ncols, W, 1.f, st));
		ST_TRY(yalm_head_norm_rope_append_rows(P, ldp, L.o_q, L.o_k, L.o_v, nqv, nkv, m.kv_heads, m.dim, m.vdim, L.qnorm, L.knorm, L.rot_freq, L.rot_mag,
		                                       m.rot.dims, m.rot.interleaved ? 1 : 0, sp.norm_eps, L.kring, L.vring, L.ring, L.kpool, L.vpool, keep, f32, n, pos0,
		                                       ctl, st));
		// many rows over bf16 rings: tensor-core attention; decode-sized calls, the fp32 cache and other head sizes: the SIMT kernels
		if (!f32 && n >= 16 && ldp % 4 == 0 && na % 2 == 0 && yalm_attn_window_pool_mma_shape(m.dim, m.vdim) && !attn_mma_off())
			ST_TRY(yalm_attn_window_pool_mma_sink(S.scan, na, P + L.o_q, ldp, L.kring, L.vring, L.kpool, L.vpool, n, nqv, nkv, m.dim, m.vdim, L.ring, keep, m.window,
			                                      pool, m.scale, pos0, ctl, nullptr, m.kv_heads, st));
		else
			ST_TRY(yalm_attn_window_pool_sink(S.scan, na, P + L.o_q, ldp, L.kring, m.dim, L.vring, m.vdim, L.kpool, L.vpool, S.attn_ws, n, nqv, nkv, m.dim, m.vdim,
			                                  L.ring, keep, m.window, pool, m.scale, f32, c.max_seq_len, pos0, ctl, nullptr, m.kv_heads, st));
		ST_TRY(yalm_diff_combine_rows(S.att, no, S.scan, na, m.head_gate ? P + L.o_gate : nullptr, ldp, n, m.heads, m.vdim, L.lambda, 1.f - m.diff, sp.norm_eps, st));
	}
	// output projection, the norm on its result and the residual add: one launch for a decode row
	if (gemv_fusable(c, n, no, L.wo, S.att)) {
		ST_TRY(yalm_gemv_act_norm_residual_norm(S.x, S.y1, S.att, L.wo, L.norm1b, sp.norm_eps, no, W, dt, -1, norm_after_mixer, S.xn, S.ticket, st));
		S.xn_valid = norm_after_mixer != nullptr;
	} else {
		ST_TRY(stack_linear(*this, c, S.a16, S.y1, W, S.att, no, L.wo, n, W, no, 1.f, st));
		ST_TRY(yalm_norm_residual_rows(S.x, S.y1, W, 1, L.norm1b, 0.f, sp.norm_eps, n, W, st));
	}
	// ---- feed-forward ----
	if (f.kind == FfnSpec::Dense) {
		if (!S.xn_valid) ST_TRY(yalm_norm_shift_rows(S.xn, nullptr, S.x, L.norm2, 0, 0.f, sp.norm_eps, nullptr, nullptr, n, W, pos0, ctl, st));
		S.xn_valid = false;
		if (f.gated) {
			ST_TRY(stack_linear(*this, c, S.a16, S.gu, 2 * f.ff, S.xn, W, L.wgu, n, 2 * f.ff, W, 1.f, st));
			if (gemv_fusable(c, n, f.ff, L.wdown, S.gu) && (size_t)f.ff * 4 % 16 == 0)
				ST_TRY(yalm_gemv_norm_residual(S.x, S.y1, S.gu, L.wdown, L.norm2b, 0.f, sp.norm_eps, f.ff, W, dt, 1, glu_act_code(f.act), f.act_alpha, f.limit,
				                               f.up_offset, S.ticket, st));
			else {
				ST_TRY(yalm_glu_act_rows(S.h, S.gu, n, f.ff, glu_act_code(f.act), f.act_alpha, f.limit, f.up_offset, st));
				ST_TRY(stack_linear(*this, c, S.a16, S.y1, W, S.h, f.ff, L.wdown, n, W, f.ff, 1.f, st));
				ST_TRY(yalm_norm_residual_rows(S.x, S.y1, W, 1, L.norm2b, 0.f, sp.norm_eps, n, W, st));
			}
		} else {
			ST_TRY(stack_linear(*this, c, S.a16, S.gu, f.ff, S.xn, W, L.wgu, n, f.ff, W, 1.f, st));
			if (gemv_fusable(c, n, f.ff, L.wdown, S.gu)) { // the activation is applied while the down projection stages its input
				ST_TRY(yalm_gemv_act_norm_residual_norm(S.x, S.y1, S.gu, L.wdown, L.norm2b, sp.norm_eps, f.ff, W, dt, plain_act_code(f.act), norm_after_ffn, S.xn,
				                                        S.ticket, st));
				S.xn_valid = norm_after_ffn != nullptr;
			} else {
				ST_TRY(yalm_act_rows(S.gu, f.ff, n, f.ff, plain_act_code(f.act), st));
				ST_TRY(stack_linear(*this, c, S.a16, S.y1, W, S.gu, f.ff, L.wdown, n, W, f.ff, 1.f, st));
				ST_TRY(yalm_norm_residual_rows(S.x, S.y1, W, 1, L.norm2b, 0.f, sp.norm_eps, n, W, st));
			}
		}
	}
	// ---- token side input ----
	if (side) {
		const int sd = sp.token_side, ldt = sd * (int)sp.layers.size(), col0 = index * sd;
		const int *toks = from_ctl ? nullptr : S.tokens;
		if (sd % 8 == 0 && W % 8 == 0 && !side_one_kernel()) {
			// h = gelu_tanh(G x) * e: many rows through the tensor-core product, few as one warp per gate row; then y = P h like any product
			if (!f32 && n >= 32) {
				ST_TRY(stack_linear(*this, c, S.a16, S.gu, sd, S.x, W, L.side_gate, n, sd, W, 1.f, st));
				ST_TRY(yalm_token_side_gate_rows(S.gu, sd, nullptr, 0, _side_table, ldt, col0, toks, ctl, nullptr, dt, n, W, sd, st));
			} else
				ST_TRY(yalm_token_side_gate_rows(S.gu, sd, S.x, W, _side_table, ldt, col0, toks, ctl, L.side_gate, dt, n, W, sd, st));
			if (gemv_fusable(c, n, sd, L.side_proj, S.gu)) {
				ST_TRY(yalm_gemv_act_norm_residual_norm(S.x, S.y1, S.gu, L.side_proj, L.side_norm, sp.norm_eps, sd, W, dt, -1, norm_after_side, S.xn, S.ticket, st));
				S.xn_valid = norm_after_side != nullptr;
			} else {
				ST_TRY(stack_linear(*this, c, S.a16, S.y1, W, S.gu, sd, L.side_proj, n, W, sd, 1.f, st));
				ST_TRY(yalm_norm_residual_rows(S.x, S.y1, W, 1, L.side_norm, 0.f, sp.norm_eps, n, W, st));
			}
		} else
			ST_TRY(yalm_token_side_rows(S.x, _side_table, ldt, col0, toks, ctl, L.side_gate, L.side_proj, L.side_norm, dt, n, W, sd, sp.norm_eps, st));
	}
	return 0;
}

int Model::stack_pass(InferenceState &s, int n, int pos0, bool from_ctl, int n_want) {
	const Config &c = *config;
	const StackSpec &sp = *c.stack;
	StackScratch &S = *_scratch;
	cudaStream_t st = s.stream();
	const int dt = static_cast<int>(c.weight_dtype), W = sp.width, f32 = c.weight_dtype == DType::F32;
	const int *ctl = from_ctl ? s.ctl() : nullptr;
	const float woff = sp.norm_one_plus ? 1.f : 0.f;
	ST_TRY(yalm_embed_rows(S.x, token_embedding_table, _pos_table, dt, from_ctl ? nullptr : S.tokens, n, W, pos0, ctl, sp.embed_scale, st));
	if (sp.embed_norm) ST_TRY(yalm_norm_shift_rows(S.x, nullptr, S.x, _embed_norm, sp.norm_scalar, woff, sp.norm_eps, nullptr, nullptr, n, W, pos0, ctl, st));
	if (sp.depth_average) ST_TRY(yalm_depth_average_rows(S.x, S.hist, (size_t)S.cap * W, nullptr, 1, n, W, nullptr, nullptr, nullptr, 0, 0, st)); // slab 0: the embedding output
	int layer_no = 0;
	auto tap = [&]() -> int { // tests: the residual rows after this layer
		if (_stack_tap && !from_ctl) {
			ST_TRY(cudaMemcpyAsync(_stack_tap + (size_t)layer_no * n * W, S.x, sizeof(float) * n * W, cudaMemcpyDeviceToHost, st));
			ST_TRY(cudaStreamSynchronize(st));
		}
		++layer_no;
		return 0;
	};
	S.xn_valid = false;
	for (size_t li = 0; li < _stack.size(); ++li) {
		auto &Lp = _stack[li];
		const StackLayer &L = *Lp;
		if (sp.parallel_block) {
			ST_TRY(stack_layer_parallel(S, L, n, pos0, ctl, st));
			ST_TRY(tap());
			continue;
		}
		if (L.sandwich) {
			ST_TRY(stack_layer_sandwich(S, L, li + 1 < _stack.size() ? _stack[li + 1].get() : nullptr, layer_no, n, pos0, ctl, from_ctl, st));
			ST_TRY(tap());
			continue;
		}
		if (own_state(L)) {
			ST_TRY(stack_layer_prenorm(S, L, layer_no, n, pos0, ctl, st));
			ST_TRY(tap());
			continue;
		}
		const yalm::MixerSpec &m = L.spec.mix;
		const int nq = m.heads * m.dim, nk = m.kv_heads * m.dim, nv = m.kv_heads * m.vdim, no = m.heads * m.vdim, ld = nq + nk + nv;
		// ---- token mixer ----
		if (gemv_fusable(c, n, W, L.wqkv, S.x)) {
			ST_TRY(yalm_gemv_qkv_post(S.qkv, S.x, L.wqkv, W, dt, L.kring, L.vring, S.vfirst, L.qnorm, L.knorm, L.vmix, L.vmode, m.heads, m.kv_heads, m.dim,
			                          m.vdim, L.ring, sp.norm_eps, f32, L.kpool, L.vpool, m.pool, L.max_blocks, pos0, ctl, S.ticket, st));
		} else {
			ST_TRY(stack_linear(*this, c, S.a16, S.qkv, ld, S.x, W, L.wqkv, n, ld, W, 1.f, st));
			ST_TRY(yalm_qkv_post_rows(S.qkv, ld, L.kring, L.vring, S.vfirst, nv, L.qnorm, L.knorm, L.vmix, L.vmode, n, m.heads, m.kv_heads, m.dim, m.vdim,
			                          L.ring, sp.norm_eps, f32, pos0, ctl, st));
			if (m.pool > 0)
				ST_TRY(yalm_kv_pool_rows(L.kpool, L.vpool, L.kring, L.vring, n, m.kv_heads, m.dim, m.vdim, L.ring, m.pool, L.max_blocks, f32, pos0, ctl, st));
		}
		// many rows over bf16 rings: tensor-core attention; decode-sized calls, the fp32 cache and other head sizes: the SIMT kernel
		if (!f32 && n >= 16 && ld % 4 == 0 && no % 2 == 0 && yalm_attn_window_pool_mma_shape(m.dim, m.vdim) && !attn_mma_off())
			ST_TRY(yalm_attn_window_pool_mma(S.att, no, S.qkv, ld, L.kring, L.vring, L.kpool, L.vpool, n, m.heads, m.kv_heads, m.dim, m.vdim, L.ring,
			                                 L.max_blocks, m.window, m.pool, m.scale, pos0, ctl, st));
		else
		ST_TRY(yalm_attn_window_pool(S.att, no, S.qkv, ld, L.kring, L.vring, L.kpool, L.vpool, S.attn_ws, n, m.heads, m.kv_heads, m.dim, m.vdim, L.ring,
		                             L.max_blocks, m.window, m.pool, m.scale, f32, c.max_seq_len, pos0, ctl, st));
		if (gemv_fusable(c, n, no, L.wo, S.att))
			ST_TRY(yalm_gemv_norm_residual(S.x, S.y, S.att, L.wo, L.norm1, woff, sp.norm_eps, no, W, dt, 0, 0, 0.f, 0.f, 0.f, S.ticket, st));
		else {
			ST_TRY(stack_linear(*this, c, S.a16, S.y, W, S.att, no, L.wo, n, W, no, 1.f, st));
			ST_TRY(yalm_norm_residual_rows(S.x, S.y, W, 1, L.norm1, woff, sp.norm_eps, n, W, st));
		}
		// ---- feed-forward ----
		const FfnSpec &f = L.spec.ffn;
		const int act = f.act == yalm::GluAct::SigmoidScaled ? 2 : f.act == yalm::GluAct::Silu ? YALM_ACT_SILU : YALM_ACT_GELU;
		if (f.kind == FfnSpec::Dense) {
			ST_TRY(stack_linear(*this, c, S.a16, S.gu, 2 * f.ff, S.x, W, L.wgu, n, 2 * f.ff, W, 1.f, st));
			if (gemv_fusable(c, n, f.ff, L.wdown, S.gu) && (size_t)f.ff * 4 % 16 == 0)
				ST_TRY(yalm_gemv_norm_residual(S.x, S.y, S.gu, L.wdown, L.norm2, woff, sp.norm_eps, f.ff, W, dt, 1, act, f.act_alpha, f.limit, f.up_offset,
				                               S.ticket, st));
			else {
				ST_TRY(yalm_glu_act_rows(S.h, S.gu, n, f.ff, act, f.act_alpha, f.limit, f.up_offset, st));
				ST_TRY(stack_linear(*this, c, S.a16, S.y, W, S.h, f.ff, L.wdown, n, W, f.ff, 1.f, st));
				ST_TRY(yalm_norm_residual_rows(S.x, S.y, W, 1, L.norm2, woff, sp.norm_eps, n, W, st));
			}
		} else if (f.kind == FfnSpec::Moe) {
			ST_TRY(yalm_router_topk_rows(S.ids, S.wts, S.x, W, L.router, dt, n, f.experts, f.top, W, f.score == yalm::RouterScore::Sigmoid ? 1 : 0,
			                             f.renormalize ? 1 : 0, f.renorm_eps, f.groups, f.keep_groups, st));
			if (S.moe_gu && !from_ctl && n * f.top >= 64 && W % 8 == 0 && f.ff % 8 == 0 && !moe_grouped_off())
				ST_TRY(stack_moe_grouped(S, L, S.x, S.a16, n, act, st));
			else {
				ST_TRY(yalm_moe_glu_slots(S.h, S.x, W, L.wg, L.wu, dt, S.ids, S.wts, n, f.top, f.ff, W, act, f.act_alpha, f.limit, f.up_offset,
				                          f.weight_on_input ? 1 : 0, st));
				ST_TRY(yalm_moe_down_slots(S.y, W, S.h, L.wdown, dt, S.ids, S.wts, n, f.top, f.ff, W, f.weight_on_input ? 0 : 1, st));
			}
			ST_TRY(yalm_norm_residual_rows(S.x, S.y, W, f.top, L.norm2, woff, sp.norm_eps, n, W, st));
		}
		ST_TRY(tap());
	}
	if (n_want > 0) {
		if (sp.layer_norm)
			ST_TRY(yalm_layer_norm_gather_rows(S.xn, S.x, from_ctl ? nullptr : S.want, rms_final_weight, 1, sp.norm_eps, n_want, W, st));
		else
			ST_TRY(yalm_norm_gather_rows(S.xn, S.x, from_ctl ? nullptr : S.want, rms_final_weight, sp.norm_scalar, woff, sp.norm_eps, n_want, W, st));
		// a single wanted row lands directly where the samplers read it
		float *dst = n_want == 1 ? s.logits_dev() : S.logits;
		ST_TRY(stack_linear(*this, c, S.a16, dst, sp.vocab, S.xn, W, wcls, n_want, sp.vocab, W, sp.logit_scale, st));
		if (sp.logit_softcap > 0.f) ST_TRY(yalm_softcap_rows(dst, n_want, sp.vocab, sp.logit_softcap, st));
	}
	return (int)cudaGetLastError();
}

int Model::stack_rows(InferenceState &s, const int *tokens, int n, int pos0, const int *want, int n_want, float *logits_out, const int *targets,
                      float *probs_out) {
	if (_device != Device::CUDA || s.device() != Device::CUDA) return YALM_ENOGPU;
	const Config &c = *config;
	const int V = c.vocab_size;
	if (!tokens || n < 1 || pos0 < 0 || pos0 + n > c.max_seq_len || n_want < 0 || (n_want && !want) || (targets && !probs_out)) return YALM_EINVAL;
	if (pos0 != 0 && pos0 != _stack_pos) {
		fprintf(stderr, "yalm_b200: position %d does not continue the sequence (next is %d; 0 starts a new one)\n", pos0, _stack_pos);
		return YALM_EINVAL;
	}
	for (int i = 0; i < n; ++i)
		if (tokens[i] < 0 || tokens[i] >= V) return YALM_EINVAL;
	for (int i = 0; i < n_want; ++i)
		if (want[i] < 0 || want[i] >= n || (i && want[i] <= want[i - 1])) return YALM_EINVAL;
	StackScratch &S = *_scratch;
	cudaStream_t st = s.stream();
	std::vector<int> all;
	if (targets) { // every row's logits, for the probability of its target
		all.resize(n);
		for (int i = 0; i < n; ++i) all[i] = i;
		want = all.data(), n_want = n;
	}
	int wi = 0;
	bool have_last = false;
	for (int done = 0; done < n; done += S.cap) {
		const int m = std::min(S.cap, n - done);
		int w0 = wi;
		while (wi < n_want && want[wi] < done + m) ++wi;
		const int nw = wi - w0;
		std::vector<int> local(std::max(1, nw));
		for (int i = 0; i < nw; ++i) local[i] = want[w0 + i] - done;
		ST_TRY(cudaMemcpyAsync(S.tokens, tokens + done, sizeof(int) * m, cudaMemcpyHostToDevice, st));
		if (nw) ST_TRY(cudaMemcpyAsync(S.want, local.data(), sizeof(int) * nw, cudaMemcpyHostToDevice, st));
		if (targets) ST_TRY(cudaMemcpyAsync(S.targets, targets + done, sizeof(int) * m, cudaMemcpyHostToDevice, st));
		ST_TRY(stack_pass(s, m, pos0 + done, false, nw));
		if (nw) {
			const float *src = nw == 1 ? s.logits_dev() : S.logits;
			if (nw > 1) // the last wanted row stays where the samplers read it
				ST_TRY(cudaMemcpyAsync(s.logits_dev(), S.logits + (size_t)(nw - 1) * V, sizeof(float) * V, cudaMemcpyDeviceToDevice, st));
			if (logits_out && !targets) ST_TRY(cudaMemcpyAsync(logits_out + (size_t)w0 * V, src, sizeof(float) * nw * V, cudaMemcpyDeviceToHost, st));
			if (targets) {
				ST_TRY(yalm_token_probs(src, V, nw, S.targets, S.probs, st));
				ST_TRY(cudaMemcpyAsync(probs_out + done, S.probs, sizeof(float) * nw, cudaMemcpyDeviceToHost, st));
			}
			have_last = true;
		}
		ST_TRY(cudaStreamSynchronize(st)); // `local` and the caller's arrays are host memory
	}
	_stack_pos = pos0 + n;
	if (have_last && s.host_logits()) {
		ST_TRY(cudaMemcpyAsync(s.logits(), s.logits_dev(), sizeof(float) * V, cudaMemcpyDeviceToHost, st));
		ST_TRY(cudaStreamSynchronize(st));
	}
	return (int)cudaGetLastError();
}

int Model::forward_rows(InferenceState &s, const int *tokens, int n, int pos0, const int *want, int n_want, float *logits_out) {
	if (is_stack()) return stack_rows(s, tokens, n, pos0, want, n_want, logits_out, nullptr, nullptr);
	// .yalm models: the token loop (src/main.cpp:91-97), logits kept for the wanted rows
	if (_device != Device::CUDA || s.device() != Device::CUDA) return YALM_ENOGPU;
	if (!tokens || n < 1 || pos0 < 0 || (n_want && (!want || !logits_out))) return YALM_EINVAL;
	const bool host = s.host_logits();
	s.set_host_logits(true);
	int wi = 0;
	for (int i = 0; i < n; ++i) {
		if (tokens[i] < 0 || tokens[i] >= config->vocab_size) return YALM_EINVAL;
		const bool wanted = wi < n_want && want[wi] == i;
		forward(s, tokens[i], pos0 + i, wanted ? InferenceMode::OUTPUT_LOGITS : InferenceMode::HYDRATE_KV_CACHE);
		if (wanted) memcpy(logits_out + (size_t)wi++ * config->vocab_size, s.logits(), sizeof(float) * config->vocab_size);
	}
	s.set_host_logits(host);
	return 0;
}

void Model::end_sequence(InferenceState &) {
	_stack_pos = 0; // rings and pooled blocks are overwritten from position 0 on; nothing of the old sequence is read again
}

// Decode loop on the device: token and position live in the control block, the sampler advances them, and only the token ids
// come back.  After one eager step the step (all kernels of a pass + the sampler) is replayed as one CUDA graph.
int Model::stack_generate(InferenceState &s, int token, int pos, int n_gen, float temperature, unsigned long long seed, int *tokens_out,
                          float *logits_out, float *device_ms) {
	if (_device != Device::CUDA || s.device() != Device::CUDA) return YALM_ENOGPU;
	const Config &c = *config;
	if (n_gen < 1 || n_gen > s.tokens_capacity() || token < 0 || token >= c.vocab_size || pos < 0 || pos + n_gen > c.max_seq_len || !tokens_out ||
	    !(temperature >= 0.f) || (pos != 0 && pos != _stack_pos))
		return YALM_EINVAL;
	cudaStream_t st = s.stream();
	int h[YALM_CTL_INTS] = {token, pos, 0, pos % c.max_seq_len, std::min(pos + 1, c.max_seq_len), 0, 0, 0};
	ST_TRY(cudaMemcpyAsync(s.ctl(), h, sizeof(h), cudaMemcpyHostToDevice, st));
	ST_TRY(cudaStreamSynchronize(st));
	cudaEvent_t e0, e1;
	ST_TRY(cudaEventCreate(&e0));
	ST_TRY(cudaEventCreate(&e1));
	const bool greedy = temperature == 0.f;
	auto step = [&]() -> int {
		ST_TRY(stack_pass(s, 1, 0, true, 1));
		if (greedy) return yalm_argmax_advance(s.logits_dev(), c.vocab_size, s.ctl(), c.max_seq_len, s.tokens_dev(), st);
		return yalm_sample_advance(s.logits_dev(), c.vocab_size, s.ctl(), c.max_seq_len, s.tokens_dev(), temperature, seed, st);
	};
	// one graph per sampling mode would need the temperature and seed baked in: capture the greedy step only
	CudaGraph &g = s.greedy_graph(); // per inference state: the graph holds the state's control block and logits pointers
	const bool use_graph = greedy && !logits_out;
	ST_TRY(cudaEventRecord(e0, st));
	for (int i = 0; i < n_gen; ++i) {
		if (use_graph && g.is_created) g.launch(st);
		else {
			ST_TRY(step());
			if (logits_out)
				ST_TRY(cudaMemcpyAsync(logits_out + (size_t)i * c.vocab_size, s.logits_dev(), sizeof(float) * c.vocab_size, cudaMemcpyDeviceToHost, st));
			if (use_graph) {
				ST_TRY(cudaStreamSynchronize(st));
				ST_TRY(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
				const int rc = step();
				const cudaError_t end = cudaStreamEndCapture(st, &g.graph);
				if (rc || end != cudaSuccess) return rc ? rc : (int)end;
				size_t nodes = 0;
				if (cudaGraphGetNodes(g.graph, nullptr, &nodes) == cudaSuccess) _stack_step_nodes = (int)nodes;
				ST_TRY(cudaGraphInstantiate(&g.instance, g.graph, 0));
				g.is_created = true;
			}
		}
	}
	ST_TRY(cudaEventRecord(e1, st));
	ST_TRY(cudaMemcpyAsync(tokens_out, s.tokens_dev(), sizeof(int) * n_gen, cudaMemcpyDeviceToHost, st));
	ST_TRY(cudaStreamSynchronize(st));
	if (device_ms) ST_TRY(cudaEventElapsedTime(device_ms, e0, e1));
	cudaEventDestroy(e0), cudaEventDestroy(e1);
	_stack_pos = pos + n_gen;
	return (int)cudaGetLastError();
}

int Model::stack_ring_slots(int layer) const {
	return layer >= 0 && layer < (int)_stack.size() ? _stack[layer]->ring : -1;
}

int Model::stack_read(int layer, int which, float *dst, size_t count) {
	if (layer < 0 || layer >= (int)_stack.size() || !dst || which < 0 || which > 3) return YALM_EINVAL;
	const StackLayer &L = *_stack[layer];
	const yalm::MixerSpec &m = L.spec.mix;
	ST_TRY(cudaDeviceSynchronize());
	if (which >= 2) {
		if (!L.kpool) return YALM_EINVAL;
		const size_t n = (size_t)m.kv_heads * L.max_blocks * (which == 2 ? m.dim : m.vdim);
		if (count > n) return YALM_EINVAL;
		return (int)cudaMemcpy(dst, which == 2 ? L.kpool : L.vpool, count * 4, cudaMemcpyDeviceToHost);
	}
	const size_t n = (size_t)m.kv_heads * L.ring * (which == 0 ? m.dim : m.vdim);
	if (count > n) return YALM_EINVAL;
	const void *src = which == 0 ? L.kring : L.vring;
	if (config->weight_dtype == DType::F32) return (int)cudaMemcpy(dst, src, count * 4, cudaMemcpyDeviceToHost);
	std::vector<uint16_t> tmp(count);
	ST_TRY(cudaMemcpy(tmp.data(), src, count * 2, cudaMemcpyDeviceToHost));
	for (size_t i = 0; i < count; ++i) dst[i] = widen(tmp.data(), i, DType::BF16);
	return 0;
}
