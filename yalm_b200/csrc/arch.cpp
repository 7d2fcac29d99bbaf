// Model registry and the configuration readers of the layered architectures (arch.h), plus the JSON tree reader.
#include "arch.h"

#include "yalm_api.h"

#include <algorithm>
#include <cmath>
#include <cstring>

namespace yalm {

// ---- JSON ------------------------------------------------------------------------------------------------------------
namespace {
struct JCursor {
	const char *p, *end;
	int depth = 0;
	void ws() {
		while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
	}
	bool lit(const char *s) {
		const size_t n = strlen(s);
		if ((size_t)(end - p) >= n && memcmp(p, s, n) == 0) {
			p += n;
			return true;
		}
		return false;
	}
	bool string(std::string *out) {
		if (p >= end || *p != '"') return false;
		++p;
		while (p < end && *p != '"') {
			if (*p == '\\' && p + 1 < end) {
				++p;
				switch (*p) {
				case 'n': *out += '\n'; break;
				case 't': *out += '\t'; break;
				case 'r': *out += '\r'; break;
				case 'b': *out += '\b'; break;
				case 'f': *out += '\f'; break;
				case 'u': {
					if (p + 4 >= end) return false;
					const unsigned cp = (unsigned)strtoul(std::string(p + 1, p + 5).c_str(), nullptr, 16);
					p += 4;
					if (cp < 0x80) *out += (char)cp;
					else if (cp < 0x800) *out += (char)(0xC0 | (cp >> 6)), *out += (char)(0x80 | (cp & 0x3F));
					else *out += (char)(0xE0 | (cp >> 12)), *out += (char)(0x80 | ((cp >> 6) & 0x3F)), *out += (char)(0x80 | (cp & 0x3F));
					break;
				}
				default: *out += *p;
				}
				++p;
			} else {
				*out += *p++;
			}
		}
		if (p >= end) return false;
		++p;
		return true;
	}
	bool value(JValue *v) {
		if (++depth > 64) return false;
		ws();
		if (p >= end) return false;
		bool ok = true;
		if (*p == '{') {
			++p;
			v->kind = JValue::Object;
			ws();
			if (p < end && *p == '}') ++p;
			else {
				for (;;) {
					ws();
					std::string key;
					if (!string(&key)) return false;
					ws();
					if (p >= end || *p++ != ':') return false;
					v->obj.emplace_back(key, JValue());
					if (!value(&v->obj.back().second)) return false;
					ws();
					if (p < end && *p == ',') { ++p; continue; }
					if (p < end && *p == '}') { ++p; break; }
					return false;
				}
			}
		} else if (*p == '[') {
			++p;
			v->kind = JValue::Array;
			ws();
			if (p < end && *p == ']') ++p;
			else {
				for (;;) {
					v->arr.emplace_back();
					if (!value(&v->arr.back())) return false;
					ws();
					if (p < end && *p == ',') { ++p; continue; }
					if (p < end && *p == ']') { ++p; break; }
					return false;
				}
			}
		} else if (*p == '"') {
			v->kind = JValue::String;
			ok = string(&v->str);
		} else if (lit("true")) {
			v->kind = JValue::Bool, v->b = true;
		} else if (lit("false")) {
			v->kind = JValue::Bool, v->b = false;
		} else if (lit("null")) {
			v->kind = JValue::Null;
		} else {
			// strtod needs a terminated buffer: numbers are short, copy the candidate characters
			char buf[64];
			size_t n = 0;
			while (p + n < end && n < sizeof(buf) - 1 && strchr("+-0123456789.eE", p[n])) ++n;
			if (n == 0) return false;
			memcpy(buf, p, n);
			buf[n] = 0;
			char *e = nullptr;
			v->num = strtod(buf, &e);
			if (e == buf) return false;
			p += e - buf;
			v->kind = JValue::Number;
		}
		--depth;
		return ok;
	}
};
} // namespace

bool json_parse(const char *text, size_t size, JValue *out) {
	JCursor c{text, text + size};
	*out = JValue();
	if (!c.value(out)) return false;
	c.ws();
	return c.p == c.end;
}

// ---- StackSpec -------------------------------------------------------------------------------------------------------
int StackSpec::max_q_dim() const {
	int m = 0;
	for (const LayerSpec &l : layers) m = std::max(m, l.mix.heads * l.mix.dim);
	return m;
}
int StackSpec::max_kv_dim() const {
	int m = 0;
	for (const LayerSpec &l : layers) m = std::max(m, l.mix.kv_heads * l.mix.dim);
	return m;
}
int StackSpec::max_v_dim() const {
	int m = 0;
	for (const LayerSpec &l : layers) m = std::max(m, l.mix.kv_heads * l.mix.vdim);
	return m;
}
int StackSpec::max_o_dim() const {
	int m = 0;
	for (const LayerSpec &l : layers)
		m = std::max({m, l.mix.heads * l.mix.maps * l.mix.vdim, l.ssm.inner(), l.delta.heads * l.delta.vdim, l.mix.heads * l.latent.kv_rank, l.gla.heads * l.gla.vdim});
	return m;
}
int StackSpec::max_proj() const {
	int m = 0;
	for (const LayerSpec &l : layers) m = std::max(m, l.proj_width());
	return m;
}
int StackSpec::max_conv() const {
	int m = 0;
	for (const LayerSpec &l : layers) m = std::max(m, l.conv_width());
	return m;
}
int StackSpec::max_aux() const {
	int m = 0;
	for (const LayerSpec &l : layers) m = std::max(m, l.aux_width());
	return m;
}

int LayerSpec::proj_width() const {
	if (kind == MixerKind::StateSpace) return ssm.proj();
	if (kind == MixerKind::LatentAttention) // [query latent, or the queries themselves | key / value latent + shared key part (own cache only) | gate]
		return (latent.q_rank > 0 ? latent.q_rank : mix.heads * (mix.dim + latent.rot_dim)) + (latent.kv_from < 0 ? latent.kv_rank + latent.rot_dim : 0) +
		       (mix.out_gate ? mix.heads * mix.vdim : 0);
	if (kind == MixerKind::LinearAttention) return 2 * gla.heads * gla.dim + 2 * gla.heads * gla.vdim + gla.decay_rank;
	int n = mix.maps * (mix.heads + mix.kv_heads) * mix.dim + (mix.values_are_keys ? 0 : mix.kv_heads * mix.vdim) + (mix.out_gate ? mix.heads * mix.vdim : 0);
	if (mix.head_gate) n = (n + mix.heads + 3) & ~3; // one gate column per head; rows stay 16-byte multiples
	if (kind == MixerKind::Parallel) n += 2 * delta.kv_heads * delta.dim + delta.heads * delta.vdim + delta.heads + delta.decay_rank + delta.gate_rank;
	return n;
}
int LayerSpec::mixed_width() const {
	if (kind == MixerKind::StateSpace) return ssm.inner();
	if (kind == MixerKind::LinearAttention) return gla.heads * gla.vdim;
	return mix.heads * mix.vdim + (kind == MixerKind::Parallel ? delta.heads * delta.vdim : 0);
}
int LayerSpec::conv_width() const {
	if (kind == MixerKind::StateSpace) return ssm.conv_channels();
	if (kind == MixerKind::LatentAttention) return mix.heads * (mix.dim + latent.rot_dim); // the queries as projected
	return kind == MixerKind::Parallel ? 2 * delta.kv_heads * delta.dim + delta.heads * delta.vdim : 0;
}
int LayerSpec::aux_width() const {
	if (kind == MixerKind::LatentAttention) return mix.heads * (latent.kv_rank + latent.rot_dim); // the queries against the cached rows
	if (kind == MixerKind::LinearAttention) return gla.heads * gla.dim;                       // the decays
	return kind == MixerKind::Parallel ? delta.heads * delta.dim + delta.heads * delta.vdim : 0;
}
int StackSpec::max_ff() const {
	int m = 0;
	for (const LayerSpec &l : layers) m = std::max({m, l.ffn.ff, l.ffn.shared_ff});
	return m;
}

void RotarySpec::table(std::vector<float> *freqs, float *magnitude) const {
	const int half = dims / 2;
	freqs->assign(half, 0.f);
	*magnitude = 1.f;
	std::vector<double> f(half);
	for (int i = 0; i < half; ++i) f[i] = std::pow(base, -2.0 * i / dims);
	if (factor > 0.0) {
		const double pi = 3.14159265358979323846;
		auto at = [&](double turns) { return dims * std::log(original / (2.0 * pi * turns)) / (2.0 * std::log(base)); };
		const double lo = std::max(std::floor(at(fast)), 0.0), hi = std::min(std::ceil(at(slow)), (double)(dims - 1));
		for (int i = 0; i < half; ++i) {
			const double r = std::min(1.0, std::max(0.0, (i - lo) / std::max(hi - lo, 0.001)));
			f[i] = f[i] / factor * r + f[i] * (1.0 - r);
		}
		*magnitude = (float)(0.1 * std::log(factor) + 1.0);
	}
	for (int i = 0; i < half; ++i) (*freqs)[i] = (float)f[i];
}
int StackSpec::max_top() const {
	int m = 0;
	for (const LayerSpec &l : layers) m = std::max(m, l.ffn.top);
	return m;
}
int StackSpec::max_experts() const {
	int m = 0;
	for (const LayerSpec &l : layers) m = std::max(m, l.ffn.experts);
	return m;
}

// ---- Retezen ---------------------------------------------------------------------------------------------------------
// A decoder-only stack: learned absolute positions; every sublayer reads the residual stream itself and its OUTPUT is
// RMS-normalised (weights stored around zero) before it is added back; attention without rotation, with an RMS norm over
// the whole q and k projections, a sliding window plus one mean key/value per block of tokens that has left the window,
// and values blended with the first blending layer's; feed-forward either dense (gate clamped from above, up clamped
// both ways, g * sigmoid(1.702 g) * (u + 1)) or a mixture of SiLU-gated experts routed by sigmoid scores that scale the
// expert's input.
namespace {

std::string retezen_tensor(int layer, TensorRole role, int expert) {
	const std::string l = "l" + std::to_string(layer) + ".";
	const std::string e = expert >= 0 ? "e" + std::to_string(expert) + "." : "";
	switch (role) {
	case TensorRole::Embed: return "embed";
	case TensorRole::Positions: return "pos";
	case TensorRole::FinalNorm: return "final.norm";
	case TensorRole::Head: return "head";
	case TensorRole::Norm1: return l + "norm1";
	case TensorRole::Norm2: return l + "norm2";
	case TensorRole::Wq: return l + "mix.q";
	case TensorRole::Wk: return l + "mix.k";
	case TensorRole::Wv: return l + "mix.v";
	case TensorRole::Wo: return l + "mix.o";
	case TensorRole::QNorm: return l + "mix.q.norm";
	case TensorRole::KNorm: return l + "mix.k.norm";
	case TensorRole::VMix: return l + "mix.vmix";
	case TensorRole::Gate: return l + "mlp." + e + "gate";
	case TensorRole::Up: return l + "mlp." + e + "up";
	case TensorRole::Down: return l + "mlp." + e + "down";
	case TensorRole::Router: return l + "mlp.router";
	default: break;
	}
	return "";
}

int fail(const char *what) {
	fprintf(stderr, "yalm_b200: Retezen config.json: %s\n", what);
	return YALM_EFORMAT;
}

int configure_retezen(const JValue &j, Config &cfg) {
	auto spec = std::make_shared<StackSpec>();
	StackSpec &s = *spec;
	s.arch = "Retezen";
	s.width = j["width"].integer(0);
	s.vocab = j["vocab"].integer(0);
	s.max_positions = j["max_positions"].integer(0);
	s.norm_eps = (float)j["norm"]["eps"].number(1e-5);
	s.logit_scale = (float)j["logit_scale"].number(1.0);
	s.norm_one_plus = true;
	s.norm_on_output = true;
	s.learned_positions = true;
	s.tensor_name = retezen_tensor;
	if (s.width < 1 || s.vocab < 1 || s.max_positions < 1) return fail("width, vocab and max_positions must be positive");
	const JValue &layers = j["layers"];
	if (!layers.is_array() || layers.arr.empty()) return fail("'layers' must be a non-empty list");
	for (const JValue &jl : layers.arr) {
		LayerSpec L;
		if (jl["type"].string_or("") != "attention") return fail("unknown layer type (this build has: attention)");
		const JValue &m = jl["mixer"];
		L.mix.heads = m["heads"].integer(0);
		L.mix.kv_heads = m["kv_heads"].integer(L.mix.heads);
		L.mix.dim = m["dim"].integer(0);
		L.mix.vdim = m["vdim"].integer(L.mix.dim);
		L.mix.scale = (float)m["scale"].number(1.0);
		L.mix.window = m["mask"]["size"].integer(0);
		L.mix.pool = m["mask"]["pool"].integer(0);
		L.mix.qk_norm = QkNorm::WholeProjection;
		L.mix.v_mix = m["v_mix"].truthy();
		if (L.mix.heads < 1 || L.mix.kv_heads < 1 || L.mix.heads % L.mix.kv_heads || L.mix.dim < 1 || L.mix.vdim < 1 || L.mix.window < 0 ||
		    L.mix.pool < 0)
			return fail("bad mixer sizes");
		if (L.mix.window == 0) L.mix.pool = 0; // nothing ever leaves an unbounded window
		const JValue &f = jl["mlp"];
		if (f.is_object()) {
			const std::string kind = f["kind"].string_or("");
			if (kind == "dense") {
				L.ffn.kind = FfnSpec::Dense;
				L.ffn.ff = f["ff"].integer(0);
				L.ffn.act = GluAct::SigmoidScaled;
				L.ffn.act_alpha = 1.702f;
				L.ffn.limit = (float)f["limit"].number(0.0);
				L.ffn.up_offset = 1.f;
			} else if (kind == "moe") {
				L.ffn.kind = FfnSpec::Moe;
				L.ffn.ff = f["expert"]["ff"].integer(0);
				L.ffn.act = GluAct::Silu;
				L.ffn.experts = f["router"]["experts"].integer(0);
				L.ffn.top = f["router"]["top"].integer(0);
				L.ffn.score = RouterScore::Sigmoid;
				L.ffn.renormalize = false;
				L.ffn.weight_on_input = true;
				if (L.ffn.experts < 1 || L.ffn.top < 1 || L.ffn.top > L.ffn.experts) return fail("bad router sizes");
			} else
				return fail("unknown mlp kind (this build has: dense, moe)");
			if (L.ffn.ff < 1) return fail("bad feed-forward size");
		}
		s.layers.push_back(L);
	}
	// summary fields the rest of the library sizes scratch buffers and reports from
	cfg.stack = spec;
	cfg.dim = s.width;
	cfg.vocab_size = s.vocab;
	cfg.n_layers = (int)s.layers.size();
	cfg.max_seq_len = s.max_positions;
	cfg.norm_eps = s.norm_eps;
	cfg.hidden_dim = std::max(1, s.max_ff());
	cfg.n_heads = s.layers[0].mix.heads, cfg.n_kv_heads = s.layers[0].mix.kv_heads;
	cfg.head_dim = std::max(s.layers[0].mix.dim, s.layers[0].mix.vdim);
	for (const LayerSpec &l : s.layers) // scratch sizing: heads * head_dim covers every layer's q and attention output
		while (cfg.n_heads * cfg.head_dim < std::max(l.mix.heads * l.mix.dim, l.mix.heads * l.mix.vdim)) cfg.head_dim *= 2;
	cfg.rotary_dim = 0;
	cfg.n_experts = s.max_experts(), cfg.n_experts_active = s.max_top();
	return 0;
}

// ---- Fapudra ---------------------------------------------------------------------------------------------------------
// A decoder-only stack of parallel blocks: x = norm(embed[token] * scale + positions[p]); per layer ONE scalar-weight RMS
// norm h whose output both sublayers read, x += mixer(shift(h)) + experts(h), where shift blends every coordinate with the
// previous token's h.  The mixer is either a state-space recurrence or two mixers side by side: a windowed attention with
// sigmoid weights (values = keys, biased projections, learned distance bias, kept first tokens, output gate) and a gated
// delta rule with per-channel decay.  Experts: softmax router restricted to the best groups, renormalised weights on
// the outputs, clamped g * sigmoid(1.702 g) * (u + 1).  Logits pass a tanh soft cap.
std::string fapudra_tensor(int layer, TensorRole role, int expert) {
	const std::string l = "l" + std::to_string(layer) + ".", m = l + "mix.", a = m + "left.", d = m + "right.";
	const std::string e = expert >= 0 ? "e" + std::to_string(expert) + "." : "";
	switch (role) {
	case TensorRole::Embed: return "embed";
	case TensorRole::Positions: return "pos";
	case TensorRole::EmbedNorm: return "embed.norm";
	case TensorRole::FinalNorm: return "final.norm";
	case TensorRole::Head: return "head";
	case TensorRole::Norm1: return l + "norm1";
	case TensorRole::Shift: return l + "shift";
	case TensorRole::Wq: return a + "q";
	case TensorRole::Wk: return a + "k";
	case TensorRole::QBias: return a + "q.b";
	case TensorRole::KBias: return a + "k.b";
	case TensorRole::RelBias: return a + "rel";
	case TensorRole::HeadBias: return a + "pb";
	case TensorRole::OutGate: return a + "g";
	case TensorRole::Wo: return a + "o";
	case TensorRole::SsmIn: return m + "in";
	case TensorRole::SsmConv: return m + "conv";
	case TensorRole::SsmConvBias: return m + "conv.b";
	case TensorRole::SsmDtBias: return m + "dt_bias";
	case TensorRole::SsmALog: return m + "A_log";
	case TensorRole::SsmD: return m + "D";
	case TensorRole::SsmNorm: return m + "norm";
	case TensorRole::SsmOut: return m + "o";
	case TensorRole::DeltaQ: return d + "q";
	case TensorRole::DeltaK: return d + "k";
	case TensorRole::DeltaV: return d + "v";
	case TensorRole::DeltaQConv: return d + "q.conv";
	case TensorRole::DeltaKConv: return d + "k.conv";
	case TensorRole::DeltaVConv: return d + "v.conv";
	case TensorRole::DeltaBeta: return d + "b";
	case TensorRole::DeltaALog: return d + "A_log";
	case TensorRole::DeltaNorm: return d + "norm";
	case TensorRole::DeltaDecay1: return d + "a1";
	case TensorRole::DeltaDecay2: return d + "a2";
	case TensorRole::DeltaDtBias: return d + "dt_bias";
	case TensorRole::DeltaGate1: return d + "g1";
	case TensorRole::DeltaGate2: return d + "g2";
	case TensorRole::DeltaOut: return d + "o";
	case TensorRole::Gate: return l + "mlp." + e + "gate";
	case TensorRole::Up: return l + "mlp." + e + "up";
	case TensorRole::Down: return l + "mlp." + e + "down";
	case TensorRole::Router: return l + "mlp.router";
	default: break;
	}
	return "";
}

int fail_fapudra(const char *what) {
	fprintf(stderr, "yalm_b200: Fapudra config.json: %s\n", what);
	return YALM_EFORMAT;
}

int configure_fapudra(const JValue &j, Config &cfg) {
	auto spec = std::make_shared<StackSpec>();
	StackSpec &s = *spec;
	s.arch = "Fapudra";
	s.width = j["width"].integer(0);
	s.vocab = j["vocab"].integer(0);
	s.max_positions = j["max_positions"].integer(0);
	s.norm_eps = (float)j["norm"]["eps"].number(1e-5);
	s.embed_scale = (float)j["embedding"]["scale"].number(1.0);
	s.logit_softcap = (float)j["logit_softcap"].number(0.0);
	s.learned_positions = true;
	s.embed_norm = true;
	s.norm_scalar = true;
	s.parallel_block = true;
	s.token_shift = true;
	s.tensor_name = fapudra_tensor;
	if (s.width < 1 || s.vocab < 1 || s.max_positions < 1) return fail_fapudra("width, vocab and max_positions must be positive");
	const JValue &layers = j["layers"];
	if (!layers.is_array() || layers.arr.empty()) return fail_fapudra("'layers' must be a non-empty list");
	for (const JValue &jl : layers.arr) {
		LayerSpec L;
		const std::string type = jl["type"].string_or("");
		const JValue &m = jl["mixer"];
		if (type == "mamba2") {
			L.kind = MixerKind::StateSpace;
			SsmSpec &q = L.ssm;
			q.heads = m["heads"].integer(0), q.vdim = m["vdim"].integer(0), q.state = m["state"].integer(0);
			q.groups = m["groups"].integer(1), q.norm_groups = m["norm_groups"].integer(1), q.conv = m["conv"].integer(0);
			if (q.heads < 1 || q.vdim < 1 || q.state < 1 || q.groups < 1 || q.heads % q.groups || q.norm_groups < 1 || q.inner() % q.norm_groups ||
			    q.conv < 1)
				return fail_fapudra("bad mamba2 sizes");
		} else if (type == "parallel") {
			L.kind = MixerKind::Parallel;
			const JValue &a = m["left"], &d = m["right"];
			MixerSpec &x = L.mix;
			x.heads = a["heads"].integer(0), x.kv_heads = a["kv_heads"].integer(x.heads);
			x.dim = a["dim"].integer(0), x.vdim = a["vdim"].integer(x.dim);
			x.scale = (float)a["scale"].number(1.0);
			x.window = a["mask"]["size"].integer(0), x.keep_first = a["mask"]["keep_first"].integer(0);
			x.weights = AttnWeights::Sigmoid;
			x.values_are_keys = x.qk_bias = x.out_gate = true;
			x.rel_far = a["bias_max"].integer(0);
			x.rel_rows = 1; // the table's own row count is read from the checkpoint
			if (x.heads < 1 || x.kv_heads < 1 || x.heads % x.kv_heads || x.dim < 1 || x.window < 0 || x.keep_first < 0)
				return fail_fapudra("bad attention sizes");
			if (x.vdim != x.dim) return fail_fapudra("the attention's values are its keys: vdim must equal dim");
			DeltaSpec &y = L.delta;
			y.heads = d["heads"].integer(0), y.kv_heads = d["kv_heads"].integer(y.heads);
			y.dim = d["dim"].integer(0), y.vdim = d["vdim"].integer(y.dim), y.conv = d["conv"].integer(0);
			if (y.heads < 1 || y.kv_heads < 1 || y.heads % y.kv_heads || y.dim < 1 || y.vdim < 1 || y.conv < 1) return fail_fapudra("bad delta-rule sizes");
			L.left_scale = (float)m["left_scale"].number(1.0), L.right_scale = (float)m["right_scale"].number(1.0);
		} else
			return fail_fapudra("unknown layer type (this build has: mamba2, parallel)");
		const JValue &f = jl["mlp"];
		if (f.is_object()) {
			if (f["kind"].string_or("") != "moe") return fail_fapudra("unknown mlp kind (this build has: moe)");
			FfnSpec &F = L.ffn;
			F.kind = FfnSpec::Moe;
			F.ff = f["expert"]["ff"].integer(0);
			F.act = GluAct::SigmoidScaled, F.act_alpha = 1.702f, F.up_offset = 1.f;
			F.limit = (float)f["expert"]["limit"].number(0.0);
			F.experts = f["router"]["experts"].integer(0), F.top = f["router"]["top"].integer(0);
			F.groups = f["router"]["groups"]["count"].integer(1), F.keep_groups = f["router"]["groups"]["keep"].integer(F.groups);
			F.score = RouterScore::Softmax;
			F.renormalize = true, F.renorm_eps = 1e-20f;
			F.weight_on_input = false;
			if (F.ff < 1 || F.experts < 1 || F.top < 1 || F.top > F.experts || F.groups < 1 || F.experts % F.groups || F.keep_groups < 1 ||
			    F.keep_groups > F.groups || F.top > F.keep_groups * (F.experts / F.groups))
				return fail_fapudra("bad router sizes");
		}
		s.layers.push_back(L);
	}
	cfg.stack = spec;
	cfg.dim = s.width;
	cfg.vocab_size = s.vocab;
	cfg.n_layers = (int)s.layers.size();
	cfg.max_seq_len = s.max_positions;
	cfg.norm_eps = s.norm_eps;
	cfg.hidden_dim = std::max(1, s.max_ff());
	// summary fields: the first attention's head counts if there is one, and a head size that covers every mixer's width
	cfg.n_heads = cfg.n_kv_heads = 1;
	for (const LayerSpec &l : s.layers)
		if (l.kind == MixerKind::Parallel) {
			cfg.n_heads = l.mix.heads, cfg.n_kv_heads = l.mix.kv_heads;
			break;
		}
	cfg.head_dim = 8;
	while (cfg.n_heads * cfg.head_dim < std::max(s.max_q_dim(), s.max_o_dim())) cfg.head_dim *= 2;
	cfg.rotary_dim = 0;
	cfg.n_experts = s.max_experts(), cfg.n_experts_active = s.max_top();
	return 0;
}

// ---- Fegizen ---------------------------------------------------------------------------------------------------------
// A decoder-only stack of pre-norm layers, x <- x + mixer(N(x)), x <- x + ff(N(x)), with layer norms without bias; every
// sublayer reads its normed input plus a short causal convolution of it; what a layer hands on is a learned weighted sum of
// the embedding output and all layer results so far.  Mixers: latent attention (low-rank queries, one cached latent per
// position for keys and values, a shared rotated key part, YaRN-scaled interleaved rotary positions, sliding window,
// sigmoid output gate; a layer may read another layer's cache) or gated linear attention (matrix state with per-channel
// decay).  Feed-forward: dense with tanh-GELU, or SiLU experts with a softmax router whose choice adds a stored bias, whose
// last outputs are identity experts, with renormalised scaled weights and an always-on shared expert.
std::string fegizen_tensor(int layer, TensorRole role, int expert) {
	const std::string l = "l" + std::to_string(layer) + ".", m = l + "mix.", f = l + "mlp.";
	const std::string e = expert >= 0 ? "e" + std::to_string(expert) + "." : "";
	switch (role) {
	case TensorRole::Embed: return "embed";
	case TensorRole::FinalNorm: return "final.norm";
	case TensorRole::Head: return "head";
	case TensorRole::Norm1: return l + "norm1";
	case TensorRole::Norm2: return l + "norm2";
	case TensorRole::InConv1: return l + "canon1";
	case TensorRole::InConv2: return l + "canon2";
	case TensorRole::DepthWeights: return l + "dwa";
	case TensorRole::LatentDq: return m + "dq";
	case TensorRole::LatentDqNorm: return m + "dq.norm";
	case TensorRole::LatentUq: return m + "uq";
	case TensorRole::LatentDkv: return m + "dkv";
	case TensorRole::LatentDkvNorm: return m + "dkv.norm";
	case TensorRole::LatentUk: return m + "uk";
	case TensorRole::LatentUv: return m + "uv";
	case TensorRole::OutGate: return m + "g";
	case TensorRole::Wo: return m + "o";
	case TensorRole::Wq: return m + "q";
	case TensorRole::Wk: return m + "k";
	case TensorRole::Wv: return m + "v";
	case TensorRole::GlaNorm: return m + "norm";
	case TensorRole::GlaDecay1: return m + "a1";
	case TensorRole::GlaDecay2: return m + "a2";
	case TensorRole::GlaDecayBias: return m + "a2.b";
	case TensorRole::Gate: return f + e + "gate";
	case TensorRole::Up: return f + e + "up";
	case TensorRole::Down: return f + e + "down";
	case TensorRole::Router: return f + "router";
	case TensorRole::RouterBias: return f + "correction";
	case TensorRole::SharedGate: return f + "shared.gate";
	case TensorRole::SharedUp: return f + "shared.up";
	case TensorRole::SharedDown: return f + "shared.down";
	default: break;
	}
	return "";
}

int fail_fegizen(const char *what) {
	fprintf(stderr, "yalm_b200: Fegizen config.json: %s\n", what);
	return YALM_EFORMAT;
}

int configure_fegizen(const JValue &j, Config &cfg) {
	auto spec = std::make_shared<StackSpec>();
	StackSpec &s = *spec;
	s.arch = "Fegizen";
	s.width = j["width"].integer(0);
	s.vocab = j["vocab"].integer(0);
	// no position table bounds the context: rotary positions, windows and recurrent state
	s.max_positions = j["max_positions"].integer(1 << 20);
	s.norm_eps = (float)j["norm"]["eps"].number(1e-5);
	s.embed_scale = (float)j["embedding"]["scale"].number(1.0);
	s.logit_scale = (float)j["logit_scale"].number(1.0);
	s.layer_norm = true;
	s.input_conv = j["canon"]["taps"].integer(0);
	s.depth_average = true;
	s.tensor_name = fegizen_tensor;
	if (s.width < 1 || s.vocab < 1 || s.max_positions < 1) return fail_fegizen("width and vocab must be positive");
	if (s.input_conv < 1) return fail_fegizen("canon.taps must be positive");
	const JValue &layers = j["layers"];
	if (!layers.is_array() || layers.arr.empty()) return fail_fegizen("'layers' must be a non-empty list");
	for (const JValue &jl : layers.arr) {
		LayerSpec L;
		const std::string type = jl["type"].string_or("");
		const JValue &m = jl["mixer"];
		const int li = (int)s.layers.size();
		if (type == "latent_attention") {
			L.kind = MixerKind::LatentAttention;
			MixerSpec &x = L.mix;
			LatentSpec &y = L.latent;
			x.heads = m["heads"].integer(0), x.kv_heads = 1; // every head reads the one cached row of a position
			x.dim = m["dim"].integer(0), x.vdim = m["vdim"].integer(0);
			x.scale = (float)m["scale"].number(1.0);
			x.window = m["mask"]["size"].integer(0);
			x.out_gate = true;
			y.q_rank = m["q_rank"].integer(0), y.kv_rank = m["kv_rank"].integer(0), y.rot_dim = m["rot_dim"].integer(0);
			y.kv_from = m["kv_from"].kind == JValue::Number ? m["kv_from"].integer(-1) : -1;
			const JValue &r = m["rot"];
			y.rot.dims = r["dims"].integer(y.rot_dim), y.rot.base = r["base"].number(10000.0), y.rot.interleaved = true;
			const JValue &sc = r["scaling"];
			if (sc.is_object()) {
				y.rot.factor = sc["factor"].number(0.0), y.rot.original = sc["original"].number(0.0);
				y.rot.fast = sc["fast"].number(0.0), y.rot.slow = sc["slow"].number(0.0);
				if (!(y.rot.factor > 0.0) || !(y.rot.original > 0.0) || !(y.rot.fast > 0.0) || !(y.rot.slow > 0.0)) return fail_fegizen("bad rotary scaling");
			}
			if (x.heads < 1 || x.dim < 0 || x.vdim < 1 || x.window < 0 || y.q_rank < 1 || y.kv_rank < 1 || y.rot_dim < 0 || x.dim + y.rot_dim < 1)
				return fail_fegizen("bad latent-attention sizes");
			if (y.rot.dims < 0 || y.rot.dims % 2 || y.rot.dims > y.rot_dim || !(y.rot.base > 0.0)) return fail_fegizen("rot.dims must be even and at most rot_dim");
			if (y.kv_from >= 0) {
				if (y.kv_from >= li) return fail_fegizen("kv_from must name an earlier layer");
				const LayerSpec &o = s.layers[y.kv_from];
				if (o.kind != MixerKind::LatentAttention || o.latent.kv_from >= 0 || o.latent.kv_rank != y.kv_rank || o.latent.rot_dim != y.rot_dim)
					return fail_fegizen("kv_from must name a latent-attention layer with its own cache and the same kv_rank and rot_dim");
			}
		} else if (type == "gla" || type == "gla_2") {
			L.kind = MixerKind::LinearAttention;
			GlaSpec &g = L.gla;
			g.heads = m["heads"].integer(0), g.dim = m["dim"].integer(0), g.vdim = m["vdim"].integer(0);
			g.tau = (float)m["tau"].number(1.0);
			if (g.heads < 1 || g.dim < 1 || g.vdim < 1 || !(g.tau > 0.f)) return fail_fegizen("bad linear-attention sizes");
		} else
			return fail_fegizen("unknown layer type (this build has: latent_attention, gla, gla_2)");
		const JValue &f = jl["mlp"];
		if (f.is_object()) {
			FfnSpec &F = L.ffn;
			const std::string kind = f["kind"].string_or("");
			if (kind == "dense") {
				F.kind = FfnSpec::Dense;
				F.ff = f["ff"].integer(0);
				F.act = GluAct::GeluTanh;
			} else if (kind == "moe") {
				F.kind = FfnSpec::Moe;
				F.ff = f["expert"]["ff"].integer(0);
				F.act = GluAct::Silu;
				F.experts = f["router"]["experts"].integer(0), F.top = f["router"]["top"].integer(0);
				F.identity = f["router"]["identity"].integer(0);
				F.router_scale = (float)f["router"]["scale"].number(1.0);
				F.score = RouterScore::Softmax;
				F.renormalize = true, F.renorm_eps = 1e-20f;
				F.choice_bias = true;
				if (f["shared"].is_object()) F.shared_ff = f["shared"]["ff"].integer(0), F.shared_act = GluAct::Silu;
				if (F.experts < 0 || F.identity < 0 || F.top < 1 || F.top > F.experts + F.identity || F.shared_ff < 0 || (F.experts > 0 && F.ff < 1))
					return fail_fegizen("bad router sizes");
			} else
				return fail_fegizen("unknown mlp kind (this build has: dense, moe)");
			if (F.kind == FfnSpec::Dense && F.ff < 1) return fail_fegizen("bad feed-forward size");
		}
		s.layers.push_back(L);
	}
	cfg.stack = spec;
	cfg.dim = s.width;
	cfg.vocab_size = s.vocab;
	cfg.n_layers = (int)s.layers.size();
	cfg.max_seq_len = s.max_positions;
	cfg.norm_eps = s.norm_eps;
	cfg.hidden_dim = std::max(1, s.max_ff());
	cfg.n_heads = cfg.n_kv_heads = 1;
	for (const LayerSpec &l : s.layers)
		if (l.kind == MixerKind::LatentAttention) {
			cfg.n_heads = l.mix.heads;
			break;
		}
	cfg.head_dim = 8;
	while (cfg.n_heads * cfg.head_dim < std::max(s.max_aux(), s.max_o_dim())) cfg.head_dim *= 2;
	cfg.rotary_dim = 0;
	cfg.n_experts = s.max_experts(), cfg.n_experts_active = s.max_top();
	return 0;
}

// ---- Kiduvik ---------------------------------------------------------------------------------------------------------
// A decoder-only stack with learned absolute positions and an RMS norm before AND after every sublayer,
// x <- x + N_b(mixer(N_a(x))), x <- x + N_b(ff(N_a(x))); at the end of every layer a slice of a second token embedding,
// gated by a projection of x, is projected back, normed and added.  Mixers: latent attention with full-rank queries (one cached
// latent per position for keys and values, a shared rotated key part, half-split rotary pairs, causal, a stored sink per head in
// the softmax's denominator; a layer may read another layer's cache) or differential attention (two softmax maps per head over
// the same values, combined with a stored lambda; per-head RMS norm on q and k, YaRN-scaled half-split rotary positions on part
// of each head, sliding window with kept first tokens, grouped key / value heads, per-head norm of the difference, one sigmoid
// gate number per head).  Feed-forward: dense, not gated, with the exact GELU.
std::string kiduvik_tensor(int layer, TensorRole role, int) {
	const std::string l = "l" + std::to_string(layer) + ".", m = l + "mix.", f = l + "mlp.", sd = l + "side.";
	switch (role) {
	case TensorRole::Embed: return "embed";
	case TensorRole::Positions: return "pos";
	case TensorRole::SideEmbed: return "side.embed";
	case TensorRole::FinalNorm: return "final.norm";
	case TensorRole::Head: return "head";
	case TensorRole::Norm1: return l + "norm1";
	case TensorRole::Norm2: return l + "norm2";
	case TensorRole::Norm1Post: return l + "norm1b";
	case TensorRole::Norm2Post: return l + "norm2b";
	case TensorRole::Wq: return m + "q";
	case TensorRole::Wk: return m + "k";
	case TensorRole::Wv: return m + "v";
	case TensorRole::Wo: return m + "o";
	case TensorRole::QNorm: return m + "q.norm";
	case TensorRole::KNorm: return m + "k.norm";
	case TensorRole::OutGate: return m + "g";
	case TensorRole::DiffLq1: return m + "lq1";
	case TensorRole::DiffLk1: return m + "lk1";
	case TensorRole::DiffLq2: return m + "lq2";
	case TensorRole::DiffLk2: return m + "lk2";
	case TensorRole::LatentDkv: return m + "dkv";
	case TensorRole::LatentDkvNorm: return m + "dkv.norm";
	case TensorRole::LatentUk: return m + "uk";
	case TensorRole::LatentUv: return m + "uv";
	case TensorRole::Sink: return m + "sink";
	case TensorRole::Up: return f + "up";
	case TensorRole::Down: return f + "down";
	case TensorRole::SideGate: return sd + "gate";
	case TensorRole::SideProj: return sd + "proj";
	case TensorRole::SideNorm: return sd + "norm";
	default: break;
	}
	return "";
}

int fail_kiduvik(const char *what) {
	fprintf(stderr, "yalm_b200: Kiduvik config.json: %s\n", what);
	return YALM_EFORMAT;
}

// rot: {dims, base, scaling: {factor, original, fast, slow}} with half-split pairs
int read_rotary(const JValue &r, int default_dims, RotarySpec *out) {
	out->dims = r["dims"].integer(default_dims), out->base = r["base"].number(10000.0), out->interleaved = false;
	const JValue &sc = r["scaling"];
	if (sc.is_object()) {
		out->factor = sc["factor"].number(0.0), out->original = sc["original"].number(0.0);
		out->fast = sc["fast"].number(0.0), out->slow = sc["slow"].number(0.0);
		if (!(out->factor > 0.0) || !(out->original > 0.0) || !(out->fast > 0.0) || !(out->slow > 0.0)) return 1;
	}
	return (out->dims < 0 || out->dims % 2 || !(out->base > 0.0)) ? 1 : 0;
}

int configure_kiduvik(const JValue &j, Config &cfg) {
	auto spec = std::make_shared<StackSpec>();
	StackSpec &s = *spec;
	s.arch = "Kiduvik";
	s.width = j["width"].integer(0);
	s.vocab = j["vocab"].integer(0);
	s.max_positions = j["max_positions"].integer(0);
	s.norm_eps = (float)j["norm"]["eps"].number(1e-5);
	s.learned_positions = true;
	s.sandwich_norm = true;
	s.token_side = j["token_side"].is_object() ? j["token_side"]["dim"].integer(0) : 0;
	s.tensor_name = kiduvik_tensor;
	if (s.width < 1 || s.vocab < 1 || s.max_positions < 1) return fail_kiduvik("width, vocab and max_positions must be positive");
	if (s.token_side < 0) return fail_kiduvik("token_side.dim must be positive");
	const JValue &layers = j["layers"];
	if (!layers.is_array() || layers.arr.empty()) return fail_kiduvik("'layers' must be a non-empty list");
	for (const JValue &jl : layers.arr) {
		LayerSpec L;
		const std::string type = jl["type"].string_or("");
		const JValue &m = jl["mixer"];
		const int li = (int)s.layers.size();
		MixerSpec &x = L.mix;
		x.heads = m["heads"].integer(0);
		x.dim = m["dim"].integer(0), x.vdim = m["vdim"].integer(0);
		x.scale = (float)m["scale"].number(1.0);
		if (type == "latent_attention") {
			L.kind = MixerKind::LatentAttention;
			LatentSpec &y = L.latent;
			x.kv_heads = 1; // every head reads the one cached row of a position
			x.window = 0, x.sink = true;
			y.q_rank = 0;
			y.kv_rank = m["kv_rank"].integer(0), y.rot_dim = m["rot_dim"].integer(0);
			y.kv_from = m["kv_from"].kind == JValue::Number ? m["kv_from"].integer(-1) : -1;
			if (read_rotary(m["rot"], y.rot_dim, &y.rot)) return fail_kiduvik("bad rotary constants");
			if (x.heads < 1 || x.dim < 0 || x.vdim < 1 || y.kv_rank < 1 || y.rot_dim < 0 || x.dim + y.rot_dim < 1) return fail_kiduvik("bad latent-attention sizes");
			if (y.rot.dims > y.rot_dim) return fail_kiduvik("rot.dims must be even and at most rot_dim");
			if (y.kv_from >= 0) {
				if (y.kv_from >= li) return fail_kiduvik("kv_from must name an earlier layer");
				const LayerSpec &o = s.layers[y.kv_from];
				if (o.kind != MixerKind::LatentAttention || o.latent.kv_from >= 0 || o.latent.kv_rank != y.kv_rank || o.latent.rot_dim != y.rot_dim)
					return fail_kiduvik("kv_from must name a latent-attention layer with its own cache and the same kv_rank and rot_dim");
			}
		} else if (type == "attention") {
			L.kind = MixerKind::Attention;
			x.kv_heads = m["kv_heads"].integer(x.heads);
			x.maps = 2, x.diff = (float)m["diff"].number(0.0);
			x.qk_norm = QkNorm::PerHead;
			x.head_gate = true;
			x.window = m["mask"]["size"].integer(0), x.keep_first = m["mask"]["keep_first"].integer(0);
			if (read_rotary(m["rot"], 0, &x.rot)) return fail_kiduvik("bad rotary constants");
			if (x.heads < 1 || x.kv_heads < 1 || x.heads % x.kv_heads || x.dim < 1 || x.vdim < 1 || x.window < 0 || x.keep_first < 0)
				return fail_kiduvik("bad attention sizes");
			if (x.rot.dims > x.dim) return fail_kiduvik("rot.dims must be even and at most dim");
			if (x.window == 0) x.keep_first = 0; // no window: every earlier token is visible anyway
		} else
			return fail_kiduvik("unknown layer type (this build has: latent_attention, attention)");
		const JValue &f = jl["mlp"];
		if (f.is_object()) {
			if (f["kind"].string_or("") != "dense") return fail_kiduvik("unknown mlp kind (this build has: dense)");
			FfnSpec &F = L.ffn;
			F.kind = FfnSpec::Dense, F.gated = false, F.act = GluAct::GeluErf;
			F.ff = f["ff"].integer(0);
			if (F.ff < 1) return fail_kiduvik("bad feed-forward size");
		}
		s.layers.push_back(L);
	}
	cfg.stack = spec;
	cfg.dim = s.width;
	cfg.vocab_size = s.vocab;
	cfg.n_layers = (int)s.layers.size();
	cfg.max_seq_len = s.max_positions;
	cfg.norm_eps = s.norm_eps;
	cfg.hidden_dim = std::max(1, s.max_ff());
	cfg.n_heads = s.layers[0].mix.heads, cfg.n_kv_heads = s.layers[0].mix.kv_heads;
	cfg.head_dim = 8;
	while (cfg.n_heads * cfg.head_dim < std::max({s.max_aux(), s.max_o_dim(), s.max_proj()})) cfg.head_dim *= 2;
	cfg.rotary_dim = 0;
	cfg.n_experts = 0, cfg.n_experts_active = 0;
	return 0;
}

const ArchEntry kArchs[] = {
    {"Retezen", configure_retezen},
    {"Fapudra", configure_fapudra},
    {"Fegizen", configure_fegizen},
    {"Kiduvik", configure_kiduvik},
};

} // namespace

const ArchEntry *find_arch(const std::string &name) {
	for (const ArchEntry &a : kArchs)
		if (name == a.name) return &a;
	return nullptr;
}

std::string arch_names() {
	std::string out;
	for (const ArchEntry &a : kArchs) out += (out.empty() ? "" : ", ") + std::string(a.name);
	return out;
}

} // namespace yalm
