// Model registry.  A checkpoint names its architecture (a `.yalm` file implicitly: the reference's Llama / Mistral /
// Mixtral block, src/model.cpp:17-75; a checkpoint directory through "architecture" in its config.json) and the
// registry turns the configuration into what Model needs: either the homogeneous Config fields the reference has, or
// a StackSpec — a list of layers, each with its own token mixer and feed-forward description and its own sizes.  The
// layered executor (stack.cpp) knows mechanisms and their parameters, not model names: a new design registers a
// reader that fills a StackSpec from its configuration and names its tensors.
#pragma once

#include "json.h"

#include <string>
#include <vector>

struct Config;

namespace yalm {

// Normalisation of q and k before the scores.
enum class QkNorm {
	None,
	WholeProjection, /* RMS over all heads' channels at once, one weight per channel */
	PerHead          /* RMS over each head's dim channels (each map's, with several maps), one weight of size dim shared by all heads */
};
// Gated feed-forward activations: y = act(g) * (u + up_offset), with optional clamps on g (from above) and u (both sides).
enum class GluAct {
	Silu,
	Gelu /* tanh form, the reference's rounded constant */,
	SigmoidScaled /* g * sigmoid(alpha * g) */,
	GeluTanh /* tanh form, sqrt(2 / pi) to fp32 precision */,
	GeluErf /* g Phi(g) with the exact error function */
};
// How router logits become expert scores.
enum class RouterScore { Softmax, Sigmoid };
// What a layer's token mixer is.
enum class MixerKind {
	Attention,  // MixerSpec alone
	StateSpace, // SsmSpec: a selective state-space recurrence with a scalar decay per head
	Parallel,   // two mixers side by side on the same input, added with fixed scales: attention (MixerSpec) + gated delta rule (DeltaSpec)
	LatentAttention, // MixerSpec + LatentSpec: queries, keys and values through low-rank latents; the cache holds the key / value latent
	LinearAttention  // GlaSpec: a (dim, vdim) matrix state per head with one decay per key channel
};
// How attention scores become weights.
enum class AttnWeights { Softmax, Sigmoid /* sigmoid(score + head bias), not normalised over the keys */ };

// Rotary positions: pair i of the first `dims` channels of a vector at position p turns by the angle p * f_i,
// f_i = base^(-2 i / dims).  interleaved: pair i = channels (2 i, 2 i + 1); else (i, i + dims / 2).  factor > 0 rescales the
// frequencies by wavelength (YaRN): with d(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(d(fast)), 0),
// hi = min(ceil(d(slow)), dims - 1), r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1): f_i <- f_i / factor * r_i + f_i (1 - r_i),
// and cos and sin are multiplied by 0.1 ln(factor) + 1.
struct RotarySpec {
	int dims = 0;
	double base = 10000.0;
	bool interleaved = true;
	double factor = 0.0, original = 0.0, fast = 0.0, slow = 0.0;
	// the table the kernels read: dims / 2 frequencies, and the factor on cos and sin (computed in double precision)
	void table(std::vector<float> *freqs, float *magnitude) const;
};

struct MixerSpec {
	int heads = 0, kv_heads = 0; // query head h reads key/value head h / (heads / kv_heads)
	int dim = 0, vdim = 0;       // per-head query/key size and value size
	float scale = 1.f;           // score = (q . k) * scale
	int window = 0;              // query i sees keys j with 0 <= i - j < window; 0: all earlier keys
	int pool = 0;                // > 0: beside the window, one mean key/value per block of `pool` tokens lying wholly before it
	QkNorm qk_norm = QkNorm::None;
	bool v_mix = false;          // values blended with the first v_mix layer's values of the same token
	int keep_first = 0;          // with a window: the sequence's first keep_first tokens stay visible at their true positions
	AttnWeights weights = AttnWeights::Softmax;
	bool values_are_keys = false; // no value projection: v = k as projected (vdim == dim)
	bool qk_bias = false;        // biases on the q and k projections
	bool out_gate = false;       // heads * sigmoid(Wg input) before the output projection
	int rel_rows = 0;            // > 0: a learned bias per (distance bucket, head) is added to the scaled score: distances below
	int rel_far = 0;             // rel_rows / 2 have a row each, the rest are spaced logarithmically up to rel_far, then the last row
	RotarySpec rot;              // dims > 0: rotary positions on the first dims channels of every query / key head (every map's)
	int maps = 1;                // 2: differential attention.  q and k hold two maps per head, each an attention of its own over the same
	                             // values; per head o = a_1 - lambda a_2, o / sqrt(mean o^2 + eps) (1 - diff), with
	float diff = 0.f;            // lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff from four stored vectors of size dim
	bool head_gate = false;      // every head's output times sigmoid(w_h . input), one number per head, before the output projection
	bool sink = false;           // a stored number per head joins the softmax's denominator as exp(sink_h): no key, no value, not scaled
};


// Latent attention: c_q = rms(W_dq x) w_q, q = W_uq c_q, per head [dim unrotated | rot_dim rotated]; W_dkv x = [kv_rank | rot_dim]:
// the first part RMS-normed is the latent c, the rest, rotated, is one key part shared by all heads.  Per head the unrotated
// key is W_uk c and the value W_uv c; score = (q_u . k_u + q_r . k_r) * scale.  The cache holds one row [c | k_r] per position,
// and the products with W_uk and W_uv move to the query side: score = (W_uk^T q_u) . c + q_r . k_r, out = W_uv (sum_j p_j c_j).
// kv_from >= 0: the layer has no W_dkv and reads that layer's cache rows with its own W_uk, W_uv, queries and window.
// q_rank == 0: full-rank queries, q = W_q x.
// heads, dim, vdim, scale, window and the output gate are MixerSpec's.
struct LatentSpec {
	int q_rank = 0, kv_rank = 0, rot_dim = 0, kv_from = -1;
	RotarySpec rot;
};

// Gated linear attention: per head a (dim, vdim) state S, S <- diag(a) S + k v^T, out = S^T q with q scaled by dim^(-1/2);
// a = sigmoid(W_a2 W_a1 x + b)^(1 / tau) per head and key channel; per head out is RMS-normed (one weight of size vdim),
// times silu(W_g x), then the output projection.
struct GlaSpec {
	int heads = 0, dim = 0, vdim = 0;
	float tau = 1.f;
	int decay_rank = 0; // filled from the tensors' shapes at load
};

// Selective state-space mixer (state-space duality form): one projection [z | x | B | C | dt], a short causal convolution +
// SiLU over x, B, C; per head a (state, vdim) matrix M with a scalar decay a = exp(-exp(A_log) dt): M <- a M + dt B x^T,
// read-out y = M^T C + D x; y * silu(z) is RMS-normed in norm_groups parts.
struct SsmSpec {
	int heads = 0, vdim = 0, state = 0, groups = 0, norm_groups = 1, conv = 0;
	int inner() const { return heads * vdim; }
	int conv_channels() const { return heads * vdim + 2 * groups * state; }
	int proj() const { return 2 * heads * vdim + 2 * groups * state + heads; }
};

// Gated delta rule with one decay per head and key channel: per head a (dim, vdim) matrix S,
// decay the rows, M <- diag(a) M; correct what M holds for this key, e = beta (v - M^T k), M <- M + k e^T; read out y = M^T q.  q, k (kv_heads x dim) and v (heads x vdim) pass a
// short causal convolution + SiLU; q, k are unit vectors per head; the decay and the output gate come from two-stage
// (low-rank) projections whose inner sizes are the checkpoint's.
struct DeltaSpec {
	int heads = 0, kv_heads = 0, dim = 0, vdim = 0, conv = 0;
	int decay_rank = 0, gate_rank = 0; // filled from the tensors' shapes at load
};

struct FfnSpec {
	enum Kind { None, Dense, Moe } kind = None;
	int ff = 0;                  // hidden size (per expert for Moe)
	GluAct act = GluAct::Silu;
	float act_alpha = 1.f;       // SigmoidScaled only
	float limit = 0.f;           // > 0: g = min(g, limit), u = clamp(u, -limit, limit)
	float up_offset = 0.f;
	int experts = 0, top = 0;
	RouterScore score = RouterScore::Softmax;
	bool renormalize = false;    // selected scores divided by their sum
	float renorm_eps = 0.f;      // ... plus this
	int groups = 1, keep_groups = 1; // experts form `groups` equal groups of neighbours; a group scores its best expert and only
	                             // the keep_groups best groups' experts can be chosen
	bool weight_on_input = false; // expert(w * h) instead of w * expert(h)
	int identity = 0;            // the router has experts + identity outputs; the last `identity` stand for experts that return their input
	bool choice_bias = false;    // experts are chosen by score + a stored bias per router output; the weights use the score alone
	float router_scale = 1.f;    // on the (renormalised) weights
	int shared_ff = 0;           // > 0: one more gated feed-forward of this hidden size reads every row and is added
	GluAct shared_act = GluAct::Silu;
	bool gated = true;           // false: no gate matrix, y = W_down act(W_up h)
};

struct LayerSpec {
	MixerKind kind = MixerKind::Attention;
	MixerSpec mix;
	SsmSpec ssm;
	DeltaSpec delta;
	LatentSpec latent;
	GlaSpec gla;
	float left_scale = 1.f, right_scale = 1.f; // Parallel: left_scale * attention + right_scale * delta rule
	FfnSpec ffn;
	// widths of what the layer computes per row, for scratch sizing
	int proj_width() const;    // the packed input projection
	int mixed_width() const;   // the input of the output projection(s), summed over the mixers
	int conv_width() const;    // channels that pass a short convolution
	int aux_width() const;     // second-stage projections
};

enum class TensorRole {
	Embed, Positions, FinalNorm, Head, Norm1, Norm2, Wq, Wk, Wv, Wo, QNorm, KNorm, VMix, Gate, Up, Down, Router,
	EmbedNorm, Shift, QBias, KBias, RelBias, HeadBias, OutGate,
	SsmIn, SsmConv, SsmConvBias, SsmDtBias, SsmALog, SsmD, SsmNorm, SsmOut,
	DeltaQ, DeltaK, DeltaV, DeltaQConv, DeltaKConv, DeltaVConv, DeltaBeta, DeltaALog, DeltaNorm, DeltaDecay1, DeltaDecay2, DeltaDtBias,
	DeltaGate1, DeltaGate2, DeltaOut,
	InConv1, InConv2, DepthWeights, RouterBias, SharedGate, SharedUp, SharedDown,
	LatentDq, LatentDqNorm, LatentUq, LatentDkv, LatentDkvNorm, LatentUk, LatentUv,
	GlaNorm, GlaDecay1, GlaDecay2, GlaDecayBias,
	Norm1Post, Norm2Post, Sink, DiffLq1, DiffLk1, DiffLq2, DiffLk2, SideEmbed, SideGate, SideProj, SideNorm
};

struct StackSpec {
	std::string arch;
	std::vector<LayerSpec> layers;
	int width = 0, vocab = 0, max_positions = 0;
	float norm_eps = 1e-5f;
	bool norm_one_plus = false;    // norm weights stored around zero: x / rms * (1 + w)
	bool norm_on_output = false;   // x += norm(sublayer(x)) with the sublayer reading x itself, instead of x += sublayer(norm(x))
	bool learned_positions = false; // x = embed[token] + positions[p]
	float logit_scale = 1.f;
	float embed_scale = 1.f;       // x = embed[token] * embed_scale (+ positions[p])
	bool embed_norm = false;       // ... then the model's norm with its own weight
	bool norm_scalar = false;      // a norm's weight is one number for all coordinates
	bool parallel_block = false;   // one norm per layer, mixer and feed-forward both read its output: x += mixer(h) + ff(h)
	bool token_shift = false;      // the mixer reads h + (previous token's h - h) * shift; the previous h is sequence state
	float logit_softcap = 0.f;     // > 0: logits <- cap * tanh(logits / cap)
	bool layer_norm = false;       // norms subtract the mean: (x - mean) / sqrt(variance + eps) * w, no bias
	int input_conv = 0;            // > 0: every sublayer reads h + conv(h), a causal convolution over time of this many taps on each
	                               // channel of its normed input; the last taps - 1 normed inputs of both sublayers are sequence state
	bool sandwich_norm = false;    // a norm before and after every sublayer: x += norm_b(sublayer(norm_a(x)))
	int token_side = 0;            // > 0: at the end of layer i, with e = the layer's slice [i token_side, (i + 1) token_side) of a second
	                               // embedding of the token: y = P (gelu_tanh(G x) * e), x += y / sqrt(mean y^2 + eps) * w (plain weight)
	bool depth_average = false;    // what a layer hands on is a learned weighted sum of the embedding output and all layer results so far
	// name of a tensor in the checkpoint; `expert` < 0 for tensors that are not per expert
	std::string (*tensor_name)(int layer, TensorRole role, int expert) = nullptr;

	int max_q_dim() const;  // max over layers of heads * dim
	int max_kv_dim() const; // kv_heads * dim
	int max_v_dim() const;  // kv_heads * vdim
	int max_o_dim() const;  // heads * vdim (every mixer's input of an output projection)
	int max_proj() const;   // widest packed input projection of a layer
	int max_conv() const;
	int max_aux() const;
	int max_ff() const;
	int max_top() const;
	int max_experts() const;
};

struct ArchEntry {
	const char *name;
	// Fills cfg (Config::stack and the summary fields) from a parsed config.json; returns 0 or YALM_EFORMAT.
	int (*configure)(const JValue &json, Config &cfg);
};

const ArchEntry *find_arch(const std::string &name);
// All registered names, for messages.
std::string arch_names();

} // namespace yalm
