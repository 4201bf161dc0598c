"""Mixers that keep a matrix per head as their state and carry it from token to token.

`DecayMix` (time mixing in the manner of RWKV-6): every projection reads its own blend of the present
and the previous token's input, x_s = h + (h_prev - h) * mu_s; receptance r, key k, value v (heads x dim)
and an output gate silu(W_g x_g); a decay per token, head and key channel, w = exp(-exp(W_2 tanh(W_1 x_w)
+ w_0)); per head

    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t        S_t = diag(w_t) S_(t-1) + k_t v_t^T

with the bonus u for the present token only; each head's o is brought to unit root mean square, then
times a channel weight and the gate, then the output projection.  State per sequence: the previous
token's input and S, float32.

`MatrixMemory` (the mLSTM cell of xLSTM): q = W_q h / sqrt(dim), k, v; per head a log input gate
i = cap tanh((W_i h + b_i) / cap) and a log forget gate f = log sigmoid(cap tanh((W_f h + b_f) / cap)); with
a running maximum m that starts at 0

    m_t = max(f + m_(t-1), i)     S_t = e^(f + m_(t-1) - m_t) S_(t-1) + e^(i - m_t) k v^T     n_t likewise with k
    o = S_t^T q / (max(|n_t . q|, e^(-m_t)) + 1e-6)

then the same unit norm, channel weight, sigmoid(W_g h) gate and output projection.  State: S, n, m, float32.

`GatedDecayMemory` (gated linear attention) and `ConstantDecayMemory` (lightning attention) are described at their
classes.

Decays, gates, exponentials, the state and every sum over it are float32 whatever the activation dtype;
the projections run through the runtime's products.  Both mixers run every kind of step through one
kernel that starts from the stored state (zeros for a new sequence), so a prompt in one step, in portions
or token by token gives the same numbers.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.spec import FixedStateSpec
from ..weights.loader import TensorSpec
from .base import Mixer, register_part
from .linear import Linear

SCAN_MAX_KEY_DIM = 1024             # a column's key channels are spread over the lanes of one warp (csrc/recurrent.cu)


def scan_fits(dim, value_dim):
    """True if the scan kernel takes heads of dim key channels (any number of value channels)."""
    return 1 <= dim <= SCAN_MAX_KEY_DIM and value_dim >= 1


class DecayMix(Mixer):
    prompt_capturable = True
    supports_append = True
    # From this rank on the decay network runs as two of the runtime's products; below it, in one kernel that keeps
    # the small intermediate in shared memory and everything in float (measured on B200 at rank 64, width 1,024: 86 us
    # in the one kernel against two products of about 8 us for 2,048 rows).
    PRODUCT_RANK = 32

    def __init__(self, prefix, hidden, heads, dim, rank, eps, out_dtype=None):
        self.hidden, self.heads, self.dim, self.rank, self.eps = hidden, heads, dim, rank, float(eps)
        self.size = heads * dim
        self.prefix = prefix
        self.proj = {s: Linear(prefix + s, self.size, hidden) for s in "rkvg"}
        self.out = Linear(prefix + "o", hidden, self.size)
        self.out_dtype = {None: None, "float32": torch.float32}[out_dtype]

    def children(self):
        return [*self.proj.values(), self.out]

    def tensor_specs(self):
        p, H, C = self.prefix, self.hidden, self.size
        return ([TensorSpec(f"{p}mu.{s}", (H,), "vector") for s in "rkvgw"]
                + [TensorSpec(p + "w1", (self.rank, H)), TensorSpec(p + "w2", (C, self.rank)),
                   TensorSpec(p + "w0", (C,), "vector"), TensorSpec(p + "u", (self.heads, self.dim), "vector"),
                   TensorSpec(p + "norm", (C,), "vector")])

    def bind(self, tensors, rt):
        p = self.prefix
        f32 = lambda name: tensors[p + name].to(torch.float32).contiguous()
        self.mu = torch.stack([f32("mu." + s) for s in "rkvgw"]).contiguous()
        self.w1, self.w2 = tensors[p + "w1"].contiguous(), tensors[p + "w2"].t().contiguous()     # W2 as [rank, channels]
        self.w2_rows = tensors[p + "w2"].contiguous()                                             # and as stored, for the products
        self.w0, self.u, self.norm_w = f32("w0"), f32("u"), f32("norm")
        self._bound = [self.mu, self.w1, self.w2, self.w0, self.u, self.norm_w]

    def state_spec(self):
        # the previous token's input, then S of every head
        return FixedStateSpec((self.hidden + self.heads * self.dim * self.dim,), "float32")

    def forward(self, rt, batch, x, state):
        T, C = batch.T, self.size
        mixes = torch.empty((5, T, self.hidden), dtype=x.dtype, device=x.device)
        kernels.shift_mix(mixes, x, self.mu, state.tensor, batch.tok_seq, batch.tok_pos, batch.seq_pos0, batch.seq_slot)
        r, k, v, g = (self.proj[s].apply(rt, mixes[i]) for i, s in enumerate("rkvg"))
        decay = torch.empty((T, C), dtype=torch.float32, device=x.device)
        if self.rank >= self.PRODUCT_RANK and self.rank % 8 == 0 and self.hidden % 8 == 0:
            # a rank that fills a product's tile: two products with the activation between them
            low = rt.linear(mixes[4], self.w1)
            kernels.tanh_inplace(low)
            kernels.decay_from_logits(decay, rt.linear(low, self.w2_rows, out_dtype=torch.float32), self.w0)
        else:
            kernels.lowrank_decay(decay, mixes[4], self.w1, self.w2, self.w0)
        o = torch.empty((T, C), dtype=x.dtype, device=x.device)
        kernels.matrix_scan("decay", o, r, k, v, g, decay, self.u, self.norm_w, state.tensor, self.hidden,
                            batch.seq_start, batch.seq_slot, batch.B, self.heads, self.dim, self.dim, 1.0, self.eps,
                            shift_src=x)
        return self.out.apply(rt, o, out_dtype=self.out_dtype)


class MatrixMemory(Mixer):
    prompt_capturable = True
    supports_append = True

    def __init__(self, prefix, hidden, heads, dim, value_dim, gate_cap, eps, out_dtype=None):
        self.hidden, self.heads, self.dim, self.value_dim = hidden, heads, dim, value_dim
        self.gate_cap, self.eps, self.prefix = float(gate_cap), float(eps), prefix
        self.k_size, self.v_size = heads * dim, heads * value_dim
        # q | k | v | g in one product: they all read the same rows
        self.qkvg = Linear([prefix + "q", prefix + "k", prefix + "v", prefix + "g"],
                           [self.k_size, self.k_size, self.v_size, self.v_size], hidden)
        self.gates = Linear([prefix + "i", prefix + "f"], [heads, heads], hidden)
        self.out = Linear(prefix + "o", hidden, self.v_size)
        self.out_dtype = {None: None, "float32": torch.float32}[out_dtype]

    def children(self):
        return [self.qkvg, self.gates, self.out]

    def tensor_specs(self):
        p = self.prefix
        return [TensorSpec(p + "i.b", (self.heads,), "vector"), TensorSpec(p + "f.b", (self.heads,), "vector"),
                TensorSpec(p + "norm", (self.v_size,), "vector")]

    def bind(self, tensors, rt):
        p = self.prefix
        self.gate_bias = torch.cat([tensors[p + "i.b"], tensors[p + "f.b"]]).to(torch.float32).contiguous()
        self.norm_w = tensors[p + "norm"].to(torch.float32).contiguous()
        self._bound = [self.gate_bias, self.norm_w]

    def state_spec(self):
        # per head: S (dim x value_dim), n (dim), m
        return FixedStateSpec((self.heads * (self.dim * self.value_dim + self.dim + 1),), "float32")

    def forward(self, rt, batch, x, state):
        T, KS, VS = batch.T, self.k_size, self.v_size
        proj = self.qkvg.apply(rt, x)
        gates = torch.empty((T, 2 * self.heads), dtype=torch.float32, device=x.device)
        kernels.capped_gates(gates, x, self.gates.weight, self.gate_bias, self.gate_cap)
        o = torch.empty((T, VS), dtype=x.dtype, device=x.device)
        kernels.matrix_scan("memory", o, proj[:, :KS], proj[:, KS:2 * KS], proj[:, 2 * KS:2 * KS + VS],
                            proj[:, 2 * KS + VS:], gates, None, self.norm_w, state.tensor, 0, batch.seq_start,
                            batch.seq_slot, batch.B, self.heads, self.dim, self.value_dim, self.dim ** -0.5, self.eps)
        return self.out.apply(rt, o, out_dtype=self.out_dtype)


class ConstantDecayMemory(Mixer):
    """Linear attention with one constant decay per head (lightning attention): q, k (heads x dim) and v
    (heads x value_dim) pass through silu; per head S_t = w S_(t-1) + k_t v_t^T and o_t = S_t^T q_t, with no
    other scale; all heads of a token together are brought to unit root mean square, then times a channel
    weight and sigmoid(W_g h), then the output projection.  State per sequence: S, float32."""
    prompt_capturable = True
    supports_append = True
    CHUNKED_MIN_ROWS = 128                  # shorter steps run the serial scan
    CHUNKED_MAX_SCRATCH = 256 << 20         # bytes of per-chunk states above which a step runs the serial scan

    def __init__(self, prefix, hidden, heads, dim, value_dim, decay, eps, out_dtype=None):
        if len(decay) != heads:
            raise ValueError(f"{len(decay)} decays for {heads} heads")
        self.hidden, self.heads, self.dim, self.value_dim = hidden, heads, dim, value_dim
        self.eps, self.prefix, self.decay_values = float(eps), prefix, [float(w) for w in decay]
        self.k_size, self.v_size = heads * dim, heads * value_dim
        self.qkvg = Linear([prefix + "q", prefix + "k", prefix + "v", prefix + "g"],
                           [self.k_size, self.k_size, self.v_size, self.v_size], hidden)
        self.out = Linear(prefix + "o", hidden, self.v_size)
        self.out_dtype = {None: None, "float32": torch.float32}[out_dtype]

    def children(self):
        return [self.qkvg, self.out]

    def tensor_specs(self):
        return [TensorSpec(self.prefix + "norm", (self.v_size,), "vector")]

    def bind(self, tensors, rt):
        self.norm_w = tensors[self.prefix + "norm"].to(torch.float32).contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=rt.device)
        self._bound = [self.norm_w, self.decay]

    def state_spec(self):
        return FixedStateSpec((self.heads * self.dim * self.value_dim,), "float32")

    def forward(self, rt, batch, x, state):
        T, KS, VS = batch.T, self.k_size, self.v_size
        proj = self.qkvg.apply(rt, x)
        o = torch.empty((T, VS), dtype=x.dtype, device=x.device)
        # prompts: the chunked form, unless its per-chunk states would take more scratch than a step is worth (many
        # long prompts at once, which give the serial scan enough independent work anyway)
        scratch = None
        if batch.kind != "decode" and batch.max_len >= self.CHUNKED_MIN_ROWS and kernels.lightning_chunked_fits(self.dim, self.value_dim):
            need = kernels.lightning_scratch_floats(batch.B, batch.max_len, self.heads, self.dim, self.value_dim)
            if need * 4 <= self.CHUNKED_MAX_SCRATCH:
                scratch = rt.scratch("lightning_chunks", need)
        kernels.matrix_scan("constant", o, proj[:, :KS], proj[:, KS:2 * KS], proj[:, 2 * KS:2 * KS + VS],
                            proj[:, 2 * KS + VS:], self.decay, None, self.norm_w, state.tensor, 0, batch.seq_start,
                            batch.seq_slot, batch.B, self.heads, self.dim, self.value_dim, 1.0, self.eps,
                            qkv_silu=True, norm_all_heads=True, chunk_scratch=scratch, max_len=batch.max_len)
        return self.out.apply(rt, o, out_dtype=self.out_dtype)


class GatedDecayMemory(Mixer):
    """Gated linear attention: q = W_q h / sqrt(dim), k (heads x dim) and v (heads x value_dim); a decay per token, head
    and key channel out of a low-rank network, w = sigmoid(W_2 (W_1 h) + b)^(1/tau); per head S_t = diag(w_t) S_(t-1) +
    k_t v_t^T and o_t = S_t^T q_t; each head's o is brought to unit root mean square over its value channels, times a
    weight per value channel that all heads share, times silu(W_g h), then the output projection.  State per sequence:
    S, float32, zeros at the start.  The decay (its logits, the logarithm of the sigmoid, the power) is float32."""
    prompt_capturable = True
    supports_append = True
    PRODUCT_RANK = DecayMix.PRODUCT_RANK

    def __init__(self, prefix, hidden, heads, dim, value_dim, rank, tau, eps, out_dtype=None):
        if not tau > 0:
            raise ValueError(f"GatedDecayMemory: tau {tau}")
        self.hidden, self.heads, self.dim, self.value_dim, self.rank = hidden, heads, dim, value_dim, rank
        self.tau, self.eps, self.prefix = float(tau), float(eps), prefix
        self.k_size, self.v_size = heads * dim, heads * value_dim
        self.qkvg = Linear([prefix + "q", prefix + "k", prefix + "v", prefix + "g"],
                           [self.k_size, self.k_size, self.v_size, self.v_size], hidden)
        self.out = Linear(prefix + "o", hidden, self.v_size)
        self.out_dtype = {None: None, "float32": torch.float32}[out_dtype]

    def children(self):
        return [self.qkvg, self.out]

    def tensor_specs(self):
        p = self.prefix
        return [TensorSpec(p + "a1", (self.rank, self.hidden)), TensorSpec(p + "a2", (self.k_size, self.rank)),
                TensorSpec(p + "a2.b", (self.k_size,), "vector"), TensorSpec(p + "norm", (self.value_dim,), "vector")]

    def bind(self, tensors, rt):
        p = self.prefix
        self.a1 = tensors[p + "a1"].contiguous()
        self.a2_rows = tensors[p + "a2"].contiguous()              # as stored, for the products
        self.a2 = tensors[p + "a2"].t().contiguous()               # [rank, channels], for the one-kernel form
        self.bias = tensors[p + "a2.b"].to(torch.float32).contiguous()
        self.norm_w = tensors[p + "norm"].to(torch.float32).repeat(self.heads).contiguous()     # the scan indexes head x channel
        self._bound = [self.a1, self.a2, self.bias, self.norm_w]

    def state_spec(self):
        return FixedStateSpec((self.heads * self.dim * self.value_dim,), "float32")

    def forward(self, rt, batch, x, state):
        T, KS, VS = batch.T, self.k_size, self.v_size
        proj = self.qkvg.apply(rt, x)
        decay = torch.empty((T, KS), dtype=torch.float32, device=x.device)
        if self.rank >= self.PRODUCT_RANK and self.rank % 8 == 0 and self.hidden % 8 == 0:
            low = rt.linear(x, self.a1)
            kernels.decay_from_logits(decay, rt.linear(low, self.a2_rows, out_dtype=torch.float32), self.bias, tau=self.tau)
        else:
            kernels.lowrank_decay(decay, x, self.a1, self.a2, self.bias, tau=self.tau)
        o = torch.empty((T, VS), dtype=x.dtype, device=x.device)
        kernels.matrix_scan("gated", o, proj[:, :KS], proj[:, KS:2 * KS], proj[:, 2 * KS:2 * KS + VS],
                            proj[:, 2 * KS + VS:], decay, None, self.norm_w, state.tensor, 0, batch.seq_start,
                            batch.seq_slot, batch.B, self.heads, self.dim, self.value_dim, self.dim ** -0.5, self.eps)
        return self.out.apply(rt, o, out_dtype=self.out_dtype)


register_part("mixer", "decay_mix", DecayMix)
register_part("mixer", "gated_decay_memory", GatedDecayMemory)
register_part("mixer", "constant_decay_memory", ConstantDecayMemory)
register_part("mixer", "matrix_memory", MatrixMemory)
