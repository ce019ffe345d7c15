"""Descriptions of a model as data: which parts, of which sizes, in which order.

A ``ModelSpec`` is what an architecture's ``model_spec(config)`` returns.  It plays
the role of vt-transformer's graph text (v1/models/qwen2-7b/inference_fp16.dag), whose
words take their constants as arguments (``RMS_EPS`` at :290, ``ROTARY_BASE`` at :39):
every part below carries its own sizes and constants, the blocks are chosen one by one,
and the order of runs is a list.  No spec names a model.

Each spec has a ``kind``: the key under which its implementation is registered
(``parts.base.register_part``).  A new kind of mixer, feed-forward, norm, position
encoding or block is a new spec class with a new ``kind`` and a class registered
for it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """``rmsnorm``: w * x / sqrt(mean(x^2) + eps).  ``layernorm``: w * (x - mean) / sqrt(var + eps), var the mean of
    the squared deviations, no bias.  ``weight_suffix`` is appended to the part's prefix for the weight's name.
    ``one_plus``: the stored weight lies around zero and multiplies as 1 + w.
    ``groups`` (``rmsnorm``): the vector is cut into that many equal consecutive parts and each is divided by its own
    root mean square; the weight [size] multiplies the whole."""
    size: int
    eps: float
    kind: str = "rmsnorm"
    weight_suffix: str = ".weight"
    one_plus: bool = False
    groups: int = 1


@dataclass(frozen=True)
class PositionSpec:
    """``rotary``: rotation of pairs (i, i + dim/2) by pos * base^(-2i/dim), cos and sin from a table of
    ``max_positions`` rows.  ``rotary_computed``: the same rotation of the first ``dim`` dimensions of a head (the
    others pass), the angle formed in 32-bit from the position where it is used: no table, no limit of positions.
    ``none``: nothing.
    ``scaling`` (``rotary_computed``): (factor, low, high, original).  A frequency f with wavelength l = 2 pi / f is kept
    where l < original / high, divided by factor where l > original / low, and between the two it is
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low).
    ``rotary_interleaved``: pairs (2i, 2i + 1) of the first ``dim`` dimensions, angle formed where it is used as for
    ``rotary_computed``.  ``ramp`` (``rotary_interleaved`` and ``rotary_computed``) = (factor, original, fast, slow): with n(t) = dim ln(original / (2 pi t)) / (2 ln base),
    lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)), dim - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    pair i turns with f_i / factor * r_i + f_i (1 - r_i), and cos and sin are multiplied by 0.1 ln(factor) + 1."""
    dim: int = 0
    base: float = 0.0
    max_positions: int = 0
    kind: str = "rotary"
    scaling: Optional[Tuple[float, float, float, float]] = None
    ramp: Optional[Tuple[float, float, float, float]] = None


@dataclass(frozen=True)
class MixerSpec:
    kind: str = "none"


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    """Grouped-query attention over a paged cache of keys and values.

    ``window``: None sees all earlier keys; w sees key j from position p if p - w < j <= p.
    ``names``: tensor names of the q, k, v and o projections below the part's prefix.
    """
    hidden: int = 0
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    qkv_bias: bool = True
    out_bias: bool = False
    window: Optional[int] = None
    scale: Optional[float] = None          # None: 1 / sqrt(head_dim)
    position: PositionSpec = field(default_factory=lambda: PositionSpec(kind="none"))
    names: Tuple[str, str, str, str] = ("q_proj", "k_proj", "v_proj", "o_proj")
    weight_suffix: str = ".weight"         # appended to a projection's name for its matrix (".bias" for its bias)
    v_dim: Optional[int] = None            # size of a head's value where it differs from head_dim (its keys' and queries')
    qk_norm_eps: Optional[float] = None    # e: after the rotation q and k are divided, head by head, by sqrt(mean(.^2) + e)
    chunk: Optional[int] = None            # c: key j is seen from position p only if j // c == p // c (counted from position 0)
    keep_first: int = 0                    # n: beside the window's keys a token sees the keys at positions below n
    bias_suffix: str = ".bias"             # appended to a projection's name for its bias
    # e: before the rotation, all heads of q together (and of k) are divided by sqrt(mean(.^2) + e) over the whole
    # projection and multiplied by a weight of that size (``norm_names`` below the part's prefix)
    proj_norm_eps: Optional[float] = None
    norm_names: Tuple[str, str] = ("q.norm", "k.norm")
    q_temp: Optional[Tuple[float, int]] = None   # (c, n): q at position p is multiplied by 1 + c ln(floor((p + 1) / n) + 1)
    softcap: Optional[float] = None        # c: score <- c tanh(score / c) after the scale
    # "zero": the softmax's denominator holds one more term exp(0); "learned": exp(s_h), s [heads] the tensor ``sink_name``;
    # the term has no key and no value and is neither scaled nor capped
    sink: str = "none"
    sink_name: str = "sink"
    # "head": head h's result is multiplied by sigmoid(G h)_h, G [heads, hidden]; "element": the heads' results are
    # multiplied element by element by sigmoid(G h), G [heads * v_dim, hidden]; G is the tensor ``gate_name``
    gate: str = "none"
    gate_name: str = "g"
    kind: str = "attention"


@dataclass(frozen=True)
class DifferentialAttentionSpec(MixerSpec):
    """Grouped-query attention whose every head has ``maps`` = 2 sets of queries and keys of ``head_dim`` over one set of
    values of ``v_dim``.  q [heads, 2, head_dim] and k [kv_heads, 2, head_dim] are divided, map by map, by their root
    mean square (``norm_eps``) and multiplied by a weight [head_dim] (one for q, one for k, shared by heads and maps),
    then rotated.  Each map is a softmax attention of its own (``scale``; position p sees j <= p with p - j < ``window``
    or j < ``keep_first``); with a_1, a_2 their results and lam = exp(lq1 . lk1) - exp(lq2 . lk2) + ``diff`` (four
    vectors [head_dim], one number a layer): o = (a_1 - lam a_2) / sqrt(mean(.^2) + norm_eps) * (1 - diff) for each head,
    then the output projection.  ``names``: q, k, v, o, the two norm weights, lq1, lk1, lq2, lk2."""
    hidden: int = 0
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    v_dim: int = 0
    scale: Optional[float] = None
    diff: float = 0.0
    window: Optional[int] = None
    keep_first: int = 0
    norm_eps: float = 1e-6
    position: PositionSpec = field(default_factory=lambda: PositionSpec(kind="none"))
    names: Tuple[str, ...] = ("q", "k", "v", "o", "q.norm", "k.norm", "lq1", "lk1", "lq2", "lk2")
    kind: str = "differential_attention"


@dataclass(frozen=True)
class RetentionSpec(MixerSpec):
    """Linear attention with one fixed decay for each head and no softmax or denominator.  For each head, with
    S [dim, v_dim] (32-bit, zero at the start of a request): S <- decay[h] S + (k_t / sqrt(dim)) v_t^T, o_t = S^T q_t,
    q and k rotated by their positions (``position``).  Each head's o is divided by its root mean square
    (``norm_eps``, no weight) and multiplied by silu(G h); then the output projection.  ``names``: q, k, v, gate,
    output."""
    hidden: int = 0
    heads: int = 0
    dim: int = 0
    v_dim: int = 0
    decay: Tuple[float, ...] = ()
    norm_eps: float = 1e-6
    position: PositionSpec = field(default_factory=lambda: PositionSpec(kind="none"))
    names: Tuple[str, ...] = ("q", "k", "v", "g", "o")
    kind: str = "retention"


@dataclass(frozen=True)
class LatentAttentionSpec(MixerSpec):
    """Softmax attention whose keys and values are made from one narrow latent a token, which is all that is kept.
    c_q = N(D_q h) (root mean square ``norm_eps``, weight), q = U_q c_q laid out head by head as [``head_dim`` plain |
    ``rot_dim`` rotated].  D_kv h has ``kv_rank`` + ``rot_dim`` rows: the first, normed the same way, are the latent c; the
    others, rotated and not normed, are a key part that all heads share.  Head i's key is [U_k,i c | shared part], its value
    U_v,i c (``v_dim``); score = q . k * ``scale``; causal softmax, with ``sink`` one more term exp(s_i) (a number a head) in
    the denominator; with ``gate`` the heads' results are multiplied by sigmoid(G h); then the output projection.
    ``names``: D_q, its norm, U_q, D_kv, its norm, U_k, U_v, output, sink, gate."""
    hidden: int = 0
    heads: int = 0
    head_dim: int = 0
    rot_dim: int = 0
    v_dim: int = 0
    q_rank: int = 0
    kv_rank: int = 0
    scale: float = 1.0
    sink: bool = False
    gate: bool = False
    norm_eps: float = 1e-6
    position: PositionSpec = field(default_factory=lambda: PositionSpec(kind="none"))
    names: Tuple[str, ...] = ("dq", "dq.norm", "uq", "dkv", "dkv.norm", "uk", "uv", "o", "sink", "g")
    kind: str = "latent_attention"


@dataclass(frozen=True)
class LightningSpec(MixerSpec):
    """Linear attention with one fixed decay a head over activated projections: q = silu(Q h), k = silu(K h),
    v = silu(V h); for each head S [dim, v_dim] (32-bit, zero at the start of a request): S <- decay[h] S + k_t v_t^T,
    o_t = S^T q_t, no other scale.  The heads' results together are divided by their root mean square (``norm_eps``),
    multiplied by a weight [heads * v_dim] and by sigmoid(G h); then the output projection.  ``names``: q, k, v, gate,
    output, the norm's weight."""
    hidden: int = 0
    heads: int = 0
    dim: int = 0
    v_dim: int = 0
    decay: Tuple[float, ...] = ()
    norm_eps: float = 1e-6
    names: Tuple[str, ...] = ("q", "k", "v", "g", "o", "norm")
    kind: str = "lightning"


@dataclass(frozen=True)
class GatedLinearAttentionSpec(MixerSpec):
    """Linear attention with a decay for every key channel.  For each head, with S [dim, v_dim] (32-bit, zero at the
    start of a request): S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T (q_t / sqrt(dim)), where
    alpha = sigmoid(z)^(1 / tau) and z = A2 (A1 h) + b is a low-rank function of the input.  Each head's o is divided
    by its root mean square (``norm_eps``) and multiplied by a weight [v_dim] shared by the heads and by
    silu(G h); then the output projection.  ``names``: q, k, v, gate, output, the norm's weight, the two low-rank
    matrices and the bias of the second."""
    hidden: int = 0
    heads: int = 0
    dim: int = 0
    v_dim: int = 0
    tau: float = 1.0
    norm_eps: float = 1e-6
    names: Tuple[str, ...] = ("q", "k", "v", "g", "o", "norm", "a1", "a2", "a2.b")
    kind: str = "gla"


@dataclass(frozen=True)
class DeltaRuleSpec(MixerSpec):
    """The generalized delta rule.  For each head, with S [dim, dim] (32-bit, zero at the start of a request) and
    u = k / sqrt(sum(k^2) + key_eps): S <- diag(w_t) S - (a_t * u_t)(u_t^T S) + k_t v_t^T (both terms read the old
    S), o_t = S^T r_t, where w = exp(-decay_rate * sigmoid(W2 tanh(W1 h) + w0)) and a = sigmoid(A h + b) per head and
    key channel.  Each head's o is divided by its root mean square (``norm_eps``); the heads together are multiplied
    by a weight [heads * dim] and by sigmoid(G h); then the output projection.  ``names``: r, k, v, gate, output, the
    norm's weight, the removal rate's matrix and bias, the decay's two low-rank matrices and its bias."""
    hidden: int = 0
    heads: int = 0
    dim: int = 0
    decay_rate: float = 0.6065306597126334     # exp(-1/2)
    key_eps: float = 1e-6
    norm_eps: float = 1e-6
    names: Tuple[str, ...] = ("r", "k", "v", "g", "o", "norm", "a", "a.b", "w1", "w2", "w0")
    kind: str = "delta_rule"


@dataclass(frozen=True)
class GatedDeltaSpec(MixerSpec):
    """The delta rule with one decay a head.  q = Q h and k = K h have ``kv_heads`` heads of ``dim``, v = V h has ``heads``
    heads of ``v_dim``; head h reads q/k head h // (heads / kv_heads).  Each of q, k, v passes a causal convolution over
    time, channel by channel (``taps`` taps, the last one the present token's, zeros before a request's first token, no bias;
    the tensor's name + ``conv_suffix``, [channels, taps]) and silu.  Then q and k are divided, head by head, by
    sqrt(sum(.^2) + ``key_eps``) and q is multiplied by dim^(-1/2).  With beta = sigmoid(B h) and
    g = exp(-exp(A_log[h]) softplus(A h + dt_bias[h])), one number a head each, and S [dim, v_dim] (32-bit, zero at the start
    of a request): S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  Each head's o is divided by its root mean
    square (``norm_eps``), multiplied by a weight [v_dim] shared by the heads and by silu(G h); then the output projection.
    A request keeps S and the last taps - 1 inputs of the convolutions.  ``names``: q, k, v, gate, output, the norm's
    weight, B, A, A_log, dt_bias."""
    hidden: int = 0
    heads: int = 0
    kv_heads: int = 0
    dim: int = 0
    v_dim: int = 0
    taps: int = 1
    key_eps: float = 1e-6
    norm_eps: float = 1e-6
    names: Tuple[str, ...] = ("q", "k", "v", "g", "o", "norm", "b", "a", "A_log", "dt_bias")
    conv_suffix: str = ".conv"
    kind: str = "gated_delta"


@dataclass(frozen=True)
class MatrixMemorySpec(MixerSpec):
    """A matrix of memory a head with exponential gates.  q = Q h dim^(-1/2), k = K h (``heads`` heads of ``dim``), v = V h
    (``v_dim``); the logarithms of the gates, one number a head: i = c tanh((I h + b_i) / c), f = log sigmoid(c tanh((F h + b_f) / c))
    with c = ``gate_cap``.  With S [dim, v_dim], n [dim] and m (32-bit, all zero at the start of a request):
    m' = max(f + m, i); S <- exp(f + m - m') S + exp(i - m') k v^T; n likewise with k alone; m <- m';
    o = S^T q / (max(|n . q|, exp(-m)) + ``den_eps``).  Each head's o is divided by its root mean square (``norm_eps``); the heads
    together are multiplied by a weight [heads * v_dim] and by sigmoid(G h); then the output projection.  ``names``: q, k, v,
    gate, output, the norm's weight, I, F; a bias is the matrix's name + ``bias_suffix``."""
    hidden: int = 0
    heads: int = 0
    dim: int = 0
    v_dim: int = 0
    gate_cap: float = 15.0
    den_eps: float = 1e-6
    norm_eps: float = 1e-6
    names: Tuple[str, ...] = ("q", "k", "v", "g", "o", "norm", "i", "f")
    bias_suffix: str = ".b"
    kind: str = "matrix_memory"


@dataclass(frozen=True)
class NormedParallelSpec(MixerSpec):
    """Several mixers side by side on the same input, each result normed before the sum:
    sum_i scales[i] * w_i * y_i / sqrt(mean(y_i^2) + eps) with y_i = branches[i](h) after its own output projection and w_i
    [hidden] the tensor ``norm_names[i]`` below the part's prefix.  ``prefixes[i]`` is appended to the part's prefix for
    branch i's tensors."""
    hidden: int = 0
    branches: Tuple[MixerSpec, ...] = ()
    scales: Tuple[float, ...] = ()
    prefixes: Tuple[str, ...] = ()
    norm_names: Tuple[str, ...] = ()
    eps: float = 1e-6
    kind: str = "parallel_normed"


@dataclass(frozen=True)
class ParallelSpec(MixerSpec):
    """Several mixers side by side on the same input: sum_i scales[i] * branches[i](h).  ``prefixes[i]`` is appended
    to the part's prefix for branch i's tensors."""
    branches: Tuple[MixerSpec, ...] = ()
    scales: Tuple[float, ...] = ()
    prefixes: Tuple[str, ...] = ()
    kind: str = "parallel"


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str = "none"


@dataclass(frozen=True)
class GatedMLPSpec(FeedForwardSpec):
    """down(act(gate(x)) * up(x)), no biases.  ``weight_suffix`` is appended to a projection's name for its matrix."""
    hidden: int = 0
    inter: int = 0
    activation: str = "silu"
    names: Tuple[str, str, str] = ("gate_proj", "up_proj", "down_proj")
    weight_suffix: str = ".weight"
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class PolyNormMLPSpec(FeedForwardSpec):
    """down(act(up(x))), no biases, with act(z) = a N(z) + b N(z^2) + c N(z^3) + e: powers element by element, N a
    token's vector of ``inter`` values divided by its root mean square (``eps`` inside the root), and (a, b, c, e) a
    tensor of four numbers.  ``names``: up, down, the four numbers."""
    hidden: int = 0
    inter: int = 0
    eps: float = 1e-6
    names: Tuple[str, str, str] = ("up", "down", "act")
    kind: str = "polynorm_mlp"


@dataclass(frozen=True)
class XieluMLPSpec(FeedForwardSpec):
    """down(act(up(x) + b_up)) + b_down with act(z) = softplus(p) z^2 + z / 2 for z > 0 and
    (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 for z <= 0; (p, q) a tensor of two numbers.  ``names``: up, down, the
    two numbers; a bias is the matrix's name + ``bias_suffix``."""
    hidden: int = 0
    inter: int = 0
    names: Tuple[str, str, str] = ("up", "down", "act")
    bias_suffix: str = ".b"
    kind: str = "xielu_mlp"


@dataclass(frozen=True)
class ExpertsSpec(FeedForwardSpec):
    """A mixture of ``experts`` gated feed-forwards (down(silu(gate(x)) * up(x)), inner size ``inter``, no biases) of
    which a token uses the ``top`` with the largest router logits z = R x (32-bit), weighted by the softmax over the
    chosen logits; with ``shared_inter`` an expert of that inner size runs for every token and is added.  Tensors:
    ``router``, ``e<i>.gate|up|down``, ``shared.gate|up|down`` below the part's prefix.
    ``activation`` "clamped": an expert's inner vector is g sigmoid(``gate_alpha`` g) (u + 1) with g = min(gate(x), ``limit``)
    and u = clamp(up(x), -``limit``, ``limit``) (the shared expert with ``shared_limit``).  ``router_weights`` "sigmoid_share":
    the chosen experts weigh as sigmoid(z) over the chosen experts' sum of sigmoid(z) (+ 1e-20), times ``router_scale``."""
    hidden: int = 0
    experts: int = 0
    top: int = 1
    inter: int = 0
    shared_inter: Optional[int] = None
    activation: str = "silu"
    limit: float = 0.0
    shared_limit: float = 0.0
    gate_alpha: float = 1.702
    router_weights: str = "softmax"
    router_scale: float = 1.0
    names: Tuple[str, str, str] = ("gate", "up", "down")
    router_name: str = "router"
    expert_prefix: str = "e"
    shared_prefix: str = "shared."
    kind: str = "experts"


@dataclass(frozen=True)
class BlockSpec:
    """One layer.  ``prenorm``: x += mixer(norm1(x)); x += ffn(norm2(x)).  With ``ffn`` None the layer has the
    first sublayer only (and no second norm).  ``sandwich``: x += m * post1(mixer(norm1(x))); x += m * post2(ffn(norm2(x)))
    with m = ``residual_mult`` and ``post1``, ``post2`` norms of the sublayers' results.
    ``postnorm``: x <- norm1(a x + mixer(shift(x))); x <- norm2(a x + ffn(x)) with a = ``stream_scale``: the norms come
    after the sums and their result is the stream.  With ``shift_name`` the mixer reads h_t + (h_(t-1) - h_t) * mu
    (mu [hidden] the tensor of that name below the layer's prefix, h_(t-1) the previous token's x, zeros before a request's
    first token), and the layer keeps a request's last x beside what its mixer keeps.

    ``prefix`` is the tensor-name prefix of the layer; ``mixer_prefix`` and the others
    are appended to it for the parts below it."""
    mixer: MixerSpec
    ffn: Optional[FeedForwardSpec]
    norm1: NormSpec
    norm2: Optional[NormSpec]
    prefix: str
    mixer_prefix: str = "self_attn."
    ffn_prefix: str = "mlp."
    norm1_name: str = "input_layernorm"
    norm2_name: str = "post_attention_layernorm"
    kind: str = "prenorm"
    post1: Optional[NormSpec] = None
    post2: Optional[NormSpec] = None
    post1_name: str = "norm1b"
    post2_name: str = "norm2b"
    residual_mult: float = 1.0
    stream_scale: float = 1.0
    shift_name: Optional[str] = None


@dataclass(frozen=True)
class RunSpec:
    """One entry of the run order: run block ``block`` with cache slot ``cache``.

    Cache slots are numbered by the model; a slot belongs to the run that writes it.  A
    run with ``writes=False`` reads a slot that an earlier run wrote (shared keys and
    values) and stores nothing.  A block may appear in several runs, each with a slot of
    its own.  For a block whose mixer keeps several things (``Mixer.cache_spec`` returns a tuple) ``cache`` is a tuple
    of slots, one for each, in that order.  ``add_embedding``: before this run the embedding's output (the stream as it
    was before the first run) is added to the stream once more."""
    block: int
    cache: object               # None, a slot, or a tuple of slots
    writes: bool = True
    add_embedding: bool = False


@dataclass(frozen=True)
class EmbeddingSpec:
    """How token ids become the residual stream.  ``table``: x[t] = scale * table[id[t]] in 32-bit."""
    vocab: int
    hidden: int
    name: str = "model.embed_tokens.weight"
    scale: float = 1.0
    kind: str = "table"


@dataclass(frozen=True)
class HeadSpec:
    """How the stream's wanted rows become logits.  ``linear``: norm, then the product with a [vocab, hidden]
    matrix: its own (``name``), or, with ``tied_to``, the tensor of that name (the embedding's; one under ``name``
    is then allowed in the weights and not read); then logits * logit_scale and, with ``logit_cap`` c > 0,
    c * tanh(logits / c)."""
    vocab: int
    hidden: int
    norm: NormSpec
    norm_name: str = "model.norm"
    name: str = "lm_head.weight"
    tied_to: Optional[str] = None
    logit_scale: float = 1.0
    logit_cap: float = 0.0
    kind: str = "linear"


@dataclass(frozen=True)
class ModelSpec:
    """Embedding, blocks in their run order, head: each a part chosen by its spec's kind."""
    vocab: int
    hidden: int
    blocks: Tuple[BlockSpec, ...]
    order: Tuple[RunSpec, ...]
    embedding: EmbeddingSpec
    head: HeadSpec
    max_positions: int = 0
    # patterns (fnmatch) of tensor names that a checkpoint of the architecture may hold and the model does not read
    ignored: Tuple[str, ...] = ()
    # token ids at which generation ends unless a request says otherwise (from the architecture's configuration)
    eos_token_ids: Tuple[int, ...] = ()

    @staticmethod
    def default_order(n_blocks: int) -> Tuple[RunSpec, ...]:
        return tuple(RunSpec(block=i, cache=i) for i in range(n_blocks))
