"""Mixers whose memory is a matrix per head, carried from token to token: gated linear attention, the matrix
memory of xLSTM (mLSTM), retention, RWKV-style time mixing (``wkv``) and the state-space form of Mamba-2.

Both project ``q`` and ``k`` (``n_head x head_dim``, ``q`` times ``head_dim ** -0.5``), ``v`` and an
output gate ``g`` (``n_head x v_head_dim``), keep per head a state ``S`` of ``head_dim x v_head_dim``
numbers in 32-bit in the request's slot of the state pool, and read ``o_t = S_t^T q_t``.

``gated_linear_attention``: ``S_t = diag(a_t) S_(t-1) + k_t v_t^T`` with one decay per key channel,
``a = sigmoid(z) ** (1 / tau)``, ``z = W_a2 (W_a1 h) + b`` (a product of two thin matrices whose inner
size the checkpoint gives).  Every head's ``o`` is RMS-normed over its features with a gain shared by
the heads, the heads are multiplied by ``silu(g)`` and projected.

``mlstm``: scalar gates per head, ``i = cap * tanh(x_i / cap)`` and ``f = logsigmoid(cap * tanh(x_f /
cap))`` (logarithms of the input and forget gates), a running maximum ``m_t = max(f + m_(t-1), i)``
that starts at 0, ``S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k_t v_t^T``, ``n_t`` the same
with ``k_t`` alone, ``o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)``.  Every head's ``o`` is
divided by its root mean square, the concatenated heads are multiplied by a gain of their whole
size and by ``sigmoid(g)`` and projected.

Decays, gates, their exponentials, the state and the norms are 32-bit whatever the compute dtype.
The state starts at zero when a request brings its first token; nothing else distinguishes a prompt
portion from a decoded token.
"""

from __future__ import annotations

import torch

from ..cache.spec import FixedStateSpec
from .base import Mixer, register_mixer
from .spec import TensorSpec


class _MatrixMemoryMixer(Mixer):
    graph_safe = True      # launches kernels only; the state slot and the token counts are read on the device
    accepts_deferred_norm = True
    mode = ""

    def __init__(self, prefix: str, width: int, n_head: int, head_dim: int, v_head_dim: int, eps: float,
                 position=None) -> None:
        super().__init__(prefix)
        self.width, self.n_head, self.head_dim, self.v_head_dim = width, n_head, head_dim, v_head_dim
        self.eps = float(eps)
        self.qk_width, self.v_width = n_head * head_dim, n_head * v_head_dim
        self.k_off, self.v_off, self.g_off = self.qk_width, 2 * self.qk_width, 2 * self.qk_width + self.v_width
        self.fused_weight = self.out_weight = self.norm_gain = None

    def _main_specs(self):
        p, c = self.prefix, self.width
        return {p + "q": TensorSpec((self.qk_width, c), "matrix", "fan_in"),
                p + "k": TensorSpec((self.qk_width, c), "matrix", "fan_in"),
                p + "v": TensorSpec((self.v_width, c), "matrix", "fan_in"),
                p + "g": TensorSpec((self.v_width, c), "matrix", "fan_in"),
                p + "o": TensorSpec((c, self.v_width), "matrix", "fan_in_residual")}

    def _bind_main(self, tensors) -> bool:
        p = self.prefix
        rows = [tensors.get(p + n) for n in ("q", "k", "v", "g")]
        if any(r is None for r in rows):
            return False
        self.fused_weight = torch.cat(rows, dim=0).contiguous()
        self.out_weight = tensors.get(p + "o")
        self.norm_gain = tensors.get(p + "norm")      # (None for a mixer whose heads have no gain)
        return True

    def plan_step(self, batch, plan, ops) -> None:
        # the kernel set may cut prompt portions into chunks that it scans side by side
        planner = getattr(ops, "plan_memory_chunks", None)
        if planner is not None:
            planner(batch, plan, self.head_dim, self.v_head_dim, self.mode == "mlstm")

    def _finish(self, ctx, proj, memory_out, aux, residual32, per_head_gain: bool, gate_activation: str):
        gate = proj[:, self.g_off: self.g_off + self.v_width]
        heads = ctx.ops.head_norm_gate(memory_out, aux, gate, self.norm_gain, self.n_head, self.v_head_dim,
                                       self.eps, per_head_gain, gate_activation, ctx.act_dtype,
                                       positions=ctx.positions)
        ctx.ops.linear_residual(heads, self.out_weight, None, residual32)


@register_mixer("gated_linear_attention")
class GatedLinearAttention(_MatrixMemoryMixer):
    mode = "gla"
    DEFAULT_DECAY_RANK = 16      # what random-weights mode gives the two decay matrices (a checkpoint's shapes win)

    def __init__(self, prefix: str, width: int, n_head: int, head_dim: int, v_head_dim: int, tau: float,
                 eps: float, position=None) -> None:
        super().__init__(prefix, width, n_head, head_dim, v_head_dim, eps)
        self.tau = float(tau)
        self.decay_in = self.decay_out = self.decay_bias = None

    def tensor_specs(self):
        p, r = self.prefix, self.DEFAULT_DECAY_RANK
        specs = self._main_specs()
        specs[p + "norm"] = TensorSpec((self.v_head_dim,), "vector", "norm_gain")
        specs[p + "a1"] = TensorSpec((-1, self.width), "matrix", "fan_in", fill=(r, self.width))
        specs[p + "a2"] = TensorSpec((self.qk_width, -1), "matrix", "fan_in", fill=(self.qk_width, r))
        specs[p + "a2.b"] = TensorSpec((self.qk_width,), "vector", "unit_normal")
        return specs

    def bind(self, tensors) -> None:
        if not self._bind_main(tensors):
            return
        p = self.prefix
        self.decay_in, self.decay_out, self.decay_bias = tensors[p + "a1"], tensors[p + "a2"], tensors[p + "a2.b"]
        if self.decay_in.shape[0] != self.decay_out.shape[1]:
            raise ValueError(f"{p}a1 {tuple(self.decay_in.shape)} and {p}a2 {tuple(self.decay_out.shape)} "
                             "do not share their inner size")

    def cache_spec(self):
        return FixedStateSpec((self.n_head * self.v_head_dim * self.head_dim,), "float32")

    def forward(self, ctx, cache, y, residual32) -> None:
        ops = ctx.ops
        if hasattr(y, "materialize"):
            y = y.materialize()                      # three projections read the normalised rows
        proj = ops.linear(y, self.fused_weight, None, "none", ctx.act_dtype)
        thin = ops.linear(y, self.decay_in, None, "none", ctx.act_dtype)
        z = ops.linear(thin, self.decay_out, self.decay_bias, "none", torch.float32)
        out, aux = ops.matrix_memory_scan(ctx, "gla", proj, 0, self.k_off, self.v_off, self.n_head, self.head_dim,
                                          self.v_head_dim, z, self.tau, cache.state)
        self._finish(ctx, proj, out, aux, residual32, False, "silu")


@register_mixer("mlstm")
class MLSTM(_MatrixMemoryMixer):
    mode = "mlstm"

    def __init__(self, prefix: str, width: int, n_head: int, head_dim: int, v_head_dim: int, gate_cap: float,
                 eps: float, position=None) -> None:
        super().__init__(prefix, width, n_head, head_dim, v_head_dim, eps)
        self.gate_cap = float(gate_cap)
        self.gate_weight = self.gate_bias = None

    def tensor_specs(self):
        p = self.prefix
        specs = self._main_specs()
        specs[p + "norm"] = TensorSpec((self.v_width,), "vector", "norm_gain")
        for name in ("i", "f"):
            specs[p + name] = TensorSpec((self.n_head, self.width), "matrix", "fan_in")
            specs[p + name + ".b"] = TensorSpec((self.n_head,), "vector", "unit_normal")
        return specs

    def bind(self, tensors) -> None:
        if not self._bind_main(tensors):
            return
        p = self.prefix
        self.gate_weight = torch.cat([tensors[p + "i"], tensors[p + "f"]], dim=0).contiguous()
        self.gate_bias = torch.cat([tensors[p + "i.b"], tensors[p + "f.b"]], dim=0).contiguous()

    def cache_spec(self):
        # per head: head_dim x (v_head_dim + 1) numbers (the last column is the normaliser n) and the maximum m
        return FixedStateSpec((self.n_head * (self.v_head_dim + 1) * self.head_dim + self.n_head,), "float32")

    def forward(self, ctx, cache, y, residual32) -> None:
        ops = ctx.ops
        if hasattr(y, "materialize"):
            y = y.materialize()
        proj = ops.linear(y, self.fused_weight, None, "none", ctx.act_dtype)
        gates = ops.linear(y, self.gate_weight, self.gate_bias, "none", torch.float32)
        out, aux = ops.matrix_memory_scan(ctx, "mlstm", proj, 0, self.k_off, self.v_off, self.n_head, self.head_dim,
                                          self.v_head_dim, gates, self.gate_cap, cache.state)
        self._finish(ctx, proj, out, aux, residual32, True, "sigmoid")


@register_mixer("retention")
class Retention(_MatrixMemoryMixer):
    """Linear attention with one fixed decay per head and no softmax or denominator: ``S_t = a_h S_(t-1) +
    (k_t / sqrt(head_dim)) v_t^T``, ``o_t = S_t^T q_t`` (``q`` unscaled), ``decay`` the list of the heads' ``a_h``.
    Every head's ``o`` is divided by its root mean square (no gain), the heads are multiplied by ``silu(g)`` and
    projected.  The decays are 32-bit numbers worked out from the list once."""

    mode = "retention"

    def __init__(self, prefix: str, width: int, n_head: int, head_dim: int, v_head_dim: int, decay, eps: float,
                 position=None) -> None:
        super().__init__(prefix, width, n_head, head_dim, v_head_dim, eps)
        self.decay = [float(a) for a in decay]
        if len(self.decay) != n_head or not all(0.0 <= a <= 1.0 for a in self.decay):
            raise ValueError(f"decay: {n_head} numbers in 0..1, one per head (got {list(decay)!r})")
        self.decays = None

    def tensor_specs(self):
        return self._main_specs()

    def bind(self, tensors) -> None:
        if self._bind_main(tensors):
            self.decays = torch.tensor(self.decay, dtype=torch.float64).to(dtype=torch.float32,
                                                                            device=self.out_weight.device)

    def cache_spec(self):
        return FixedStateSpec((self.n_head * self.v_head_dim * self.head_dim,), "float32")

    def forward(self, ctx, cache, y, residual32) -> None:
        ops = ctx.ops
        proj = ops.linear(y, self.fused_weight, None, "none", ctx.act_dtype)
        out, aux = ops.matrix_memory_scan(ctx, "retention", proj, 0, self.k_off, self.v_off, self.n_head, self.head_dim,
                                          self.v_head_dim, None, 0.0, cache.state, head_consts=self.decays)
        self._finish(ctx, proj, out, aux, residual32, False, "silu")


@register_mixer("wkv")
class WKV(Mixer):
    """RWKV-6 style time mixing.  With ``h'`` the input of the token before (zeros for a sequence's first token), each
    of r, k, v, g, w reads its own blend ``h + (h' - h) * mu_s`` (``mu.r`` ... ``mu.w``, ``[width]`` each).  ``r``, ``k``,
    ``v`` are ``n_head x head_dim`` projections of their blends (tensors ``r``, ``k``, ``v``), the gate is
    ``silu(W_g blend_g)``, the decay per head and key channel ``w = exp(-exp(W_w2 tanh(W_w1 blend_w) + w0))`` (``w1``,
    ``w2``: two thin matrices whose inner size the checkpoint gives).  Per head ``o_t = (S_(t-1) + diag(u) k_t
    v_t^T)^T r_t`` with the bonus ``u`` ``[n_head, head_dim]`` for the current token only, then ``S_t = diag(w_t)
    S_(t-1) + k_t v_t^T``.  Every head's ``o`` is divided by its root mean square, the concatenated heads times
    ``norm``, times the gate, are projected by ``o``.

    A request's state slot holds the last input ``h`` (32-bit), then the memories.  The decays' pre-activations come
    from a projection that writes 32-bit; their exponentials, the memories and the norm are 32-bit whatever the
    compute dtype.
    """

    graph_safe = True      # launches kernels only; the state slot and the token counts are read on the device
    accepts_deferred_norm = True
    mode = "wkv"
    DEFAULT_DECAY_RANK = 16      # what random-weights mode gives the two decay matrices (a checkpoint's shapes win)
    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, prefix: str, width: int, n_head: int, head_dim: int, eps: float, position=None) -> None:
        super().__init__(prefix)
        self.width, self.n_head, self.head_dim, self.eps = width, n_head, head_dim, float(eps)
        self.inner = n_head * head_dim
        self.mu = self.weights = self.decay_in = self.decay_out = self.decay_bias = None
        self.bonus = self.norm_gain = self.out_weight = None

    def tensor_specs(self):
        p, c, n, r = self.prefix, self.width, self.inner, self.DEFAULT_DECAY_RANK
        specs = {p + "mu." + s: TensorSpec((c,), "vector", "unit_interval") for s in self.MIXES}
        for s in ("r", "k", "v", "g"):
            specs[p + s] = TensorSpec((n, c), "matrix", "fan_in")
        specs[p + "w1"] = TensorSpec((-1, c), "matrix", "fan_in", fill=(r, c))
        specs[p + "w2"] = TensorSpec((n, -1), "matrix", "fan_in", fill=(n, r))
        specs[p + "w0"] = TensorSpec((n,), "vector", "unit_normal")
        specs[p + "u"] = TensorSpec((self.n_head, self.head_dim), "vector", "unit_normal")
        specs[p + "norm"] = TensorSpec((n,), "vector", "norm_gain")
        specs[p + "o"] = TensorSpec((c, n), "matrix", "fan_in_residual")
        return specs

    def bind(self, tensors) -> None:
        p = self.prefix
        if tensors.get(p + "o") is None:
            return
        self.mu = torch.stack([tensors[p + "mu." + s] for s in self.MIXES]).contiguous()
        self.weights = [tensors[p + s] for s in ("r", "k", "v", "g")]
        self.decay_in, self.decay_out, self.decay_bias = tensors[p + "w1"], tensors[p + "w2"], tensors[p + "w0"]
        if self.decay_in.shape[0] != self.decay_out.shape[1]:
            raise ValueError(f"{p}w1 {tuple(self.decay_in.shape)} and {p}w2 {tuple(self.decay_out.shape)} "
                             "do not share their inner size")
        self.bonus = tensors[p + "u"].reshape(-1).contiguous()
        self.norm_gain, self.out_weight = tensors[p + "norm"], tensors[p + "o"]

    def cache_spec(self):
        return FixedStateSpec((self.width + self.n_head * self.head_dim * self.head_dim,), "float32")

    def plan_step(self, batch, plan, ops) -> None:
        planner = getattr(ops, "plan_memory_chunks", None)
        if planner is not None:
            planner(batch, plan, self.head_dim, self.head_dim, False)

    def forward(self, ctx, cache, y, residual32) -> None:
        ops = ctx.ops
        if hasattr(y, "materialize"):
            y = y.materialize()
        n = y.shape[0]
        blends = ops.token_shift_mix(ctx, y, self.mu, cache.state)                  # [5, tokens, width]
        ops.conv_state_update(ctx, y, 0, self.width, 2, cache.state)                # the step's last input
        proj = torch.empty((4, n, self.inner), dtype=ctx.act_dtype, device=y.device)  # planes r, k, v, g
        for i, weight in enumerate(self.weights):
            ops.linear(blends[i], weight, None, "none", ctx.act_dtype, out=proj[i])
        thin = ops.linear(blends[4], self.decay_in, None, "none", torch.float32)
        thin = ops.tanh_cast(thin, ctx.act_dtype)
        z = ops.linear(thin, self.decay_out, self.decay_bias, "none", torch.float32)
        plane = n * self.inner
        out, _ = ops.matrix_memory_scan(ctx, "wkv", proj, 0, plane, 2 * plane, self.n_head, self.head_dim, self.head_dim,
                                        z, 0.0, cache.state, state_offset=self.width, head_consts=self.bonus)
        heads = ops.head_norm_gate(out, None, proj[3], self.norm_gain, self.n_head, self.head_dim, self.eps, True, "silu",
                                   ctx.act_dtype, positions=ctx.positions)
        ops.linear_residual(heads, self.out_weight, None, residual32)


@register_mixer("state_space_duality")
class StateSpaceDuality(Mixer):
    """Mamba-2: a matrix memory per head with one scalar decay per head and step, ``inner = n_head * v_head_dim``.

    ``W_in h`` is ``[z: inner | x: inner | B: groups * state | C: groups * state | dt: n_head]``.  ``x``, ``B`` and ``C``
    together pass a causal convolution per channel (``conv`` ``[channels, taps]``, the last tap weighs the current
    token, zeros before the sequence's start; bias ``conv.b``) and silu.  ``dt <- softplus(dt + dt_bias)``.  Per head
    (head ``a`` uses the B and C of group ``a // (n_head / groups)``): ``S_t = exp(-exp(A_log_a) dt) S_(t-1) + dt B_t
    x_t^T`` (``state x v_head_dim``), ``y_t = S_t^T C_t + D_a x_t``.  The concatenated heads times ``silu(z)`` are
    RMS-normed in ``norm_groups`` equal parts, each by its own root mean square, times ``norm``, and projected.

    A request's state slot holds the last ``taps - 1`` inputs of the convolution (32-bit), then the memories.  The
    step sizes come from a projection of their own that writes 32-bit; softplus, decays, the memories and the norm
    are 32-bit whatever the compute dtype.
    """

    graph_safe = True      # launches kernels only; the state slot and the token counts are read on the device
    accepts_deferred_norm = True

    def __init__(self, prefix: str, width: int, n_head: int, v_head_dim: int, state: int, groups: int, taps: int,
                 norm_groups: int, eps: float, position=None) -> None:
        super().__init__(prefix)
        if n_head % groups or (n_head * v_head_dim) % norm_groups:
            raise ValueError("heads must form equal groups, and their features equal parts for the norm")
        self.width, self.n_head, self.v_head_dim, self.state, self.groups = width, n_head, v_head_dim, state, groups
        self.taps, self.norm_groups, self.eps = taps, norm_groups, float(eps)
        self.inner = n_head * v_head_dim
        self.channels = self.inner + 2 * groups * state          # what passes the convolution: [x | B | C]
        self.conv_state = (taps - 1) * self.channels
        self.main_weight = self.step_weight = self.step_bias = self.out_weight = None
        self.conv_taps = self.conv_bias = self.head_consts = self.norm_gain = None

    def tensor_specs(self):
        p, c = self.prefix, self.width
        return {p + "in": TensorSpec((self.inner + self.channels + self.n_head, c), "matrix", "fan_in"),
                p + "conv": TensorSpec((self.channels, self.taps), "vector", "fan_in"),
                p + "conv.b": TensorSpec((self.channels,), "vector", "norm_shift"),
                p + "dt_bias": TensorSpec((self.n_head,), "vector", "unit_normal"),
                p + "A_log": TensorSpec((self.n_head,), "vector", "unit_normal"),
                p + "D": TensorSpec((self.n_head,), "vector", "norm_gain"),
                p + "norm": TensorSpec((self.inner,), "vector", "norm_gain"),
                p + "o": TensorSpec((c, self.inner), "matrix", "fan_in_residual")}

    def bind(self, tensors) -> None:
        p = self.prefix
        w_in = tensors.get(p + "in")
        if w_in is None:
            return
        split = self.inner + self.channels
        # the step sizes get a projection of their own: it writes 32-bit and adds dt_bias on its way
        self.main_weight, self.step_weight = w_in[:split].contiguous(), w_in[split:].contiguous()
        self.step_bias = tensors[p + "dt_bias"]
        self.conv_taps, self.conv_bias = tensors[p + "conv"], tensors[p + "conv.b"]
        self.head_consts = torch.cat([tensors[p + "A_log"], tensors[p + "D"]]).contiguous()
        self.norm_gain, self.out_weight = tensors[p + "norm"], tensors[p + "o"]

    def cache_spec(self):
        return FixedStateSpec((self.conv_state + self.n_head * self.v_head_dim * self.state,), "float32")

    def plan_step(self, batch, plan, ops) -> None:
        # the kernel set may cut prompt portions into chunks that it scans side by side
        planner = getattr(ops, "plan_memory_chunks", None)
        if planner is not None:
            planner(batch, plan, self.state, self.v_head_dim, False)

    def forward(self, ctx, cache, y, residual32) -> None:
        ops = ctx.ops
        if hasattr(y, "materialize"):
            y = y.materialize()                      # two projections read the normalised rows
        proj = ops.linear(y, self.main_weight, None, "none", ctx.act_dtype)              # [z | x | B | C]
        steps = ops.linear(y, self.step_weight, self.step_bias, "none", torch.float32)   # dt + dt_bias
        xbc = ops.causal_conv_silu(ctx, proj, self.inner, self.channels, self.conv_taps, self.conv_bias, cache.state)
        ops.conv_state_update(ctx, proj, self.inner, self.channels, self.taps, cache.state)
        b_off = self.inner
        out, _ = ops.matrix_memory_scan(ctx, "ssd", xbc, b_off + self.groups * self.state, b_off, 0, self.n_head,
                                        self.state, self.v_head_dim, steps, 0.0, cache.state,
                                        state_offset=self.conv_state, qk_group=self.n_head // self.groups,
                                        head_consts=self.head_consts)
        heads = ops.gated_group_norm(out, proj[:, : self.inner], self.norm_gain, self.norm_groups, self.eps,
                                     ctx.act_dtype, positions=ctx.positions)
        ops.linear_residual(heads, self.out_weight, None, residual32)
