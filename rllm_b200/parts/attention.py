"""Grouped-query causal attention over a paged cache: the Llama mixer.

q, k, v projections without bias (one fused matrix product over the stacked
weights), head split, position encoding on q and k, write of k and v into the
run's cache pages, attention of every query token over its sequence's cache
through the block table, output projection
(crates/rllm-model/src/layers.rs:280-347 for the math, :363-571 for the paged
intent).  kv head of query head h is h // (nq // nkv)
(crates/rllm-kernels/src/cuda/paged_attention.cu:113); scores are scaled by
1/sqrt(head_dim) (layers.rs:326-329) unless ``scale`` is given.

Portions of prompts and single decoded tokens are one code path: the tokens
of this step are written to the cache first and every query then reads keys
0 .. its own position (or its window) from the cache.

Two options beyond the Llama's: ``v_dim``, a value head of another size than
a query and key head (the output projection then reads num_heads * v_dim), and
``qk_norm`` = eps: every query head and every key head is divided by its root
mean square (eps inside the root) and multiplied by a weight [head_dim] that
all heads share (tensor names "q_norm", "k_norm").  With either, the tokens'
keys (normalised) and values are written to the pages by one kernel and the
attention reads everything from there.

More options, each with its constants as parameters; a mixer with any of them goes the same way (one
kernel adds the biases, normalises, rotates and writes the pages; the attention reads from the pages: the
tcgen05 or the mma.sync kernel's form with options where keys and values have one size that it takes, else
the CUDA-core kernel; for single decoded tokens the tensor-core decode kernel does the biases, the rotation
and the cache write itself):
``bias`` True: q, k, v and the output projection have biases ("q_bias", "k_bias", "v_bias", "o_bias"),
added in float32; ``softcap`` = c: a scaled score s becomes c tanh(s / c); ``chunk`` = n: a query at
position p sees only keys j with floor(j / n) = floor(p / n), counted from the sequence's position 0;
``keep_first`` = n (with ``window``): keys 0 .. n-1 stay visible behind the window, at their true
positions; ``sinks`` True: exp(sink[h]) ("sink", one number a head) joins the softmax's denominator, with
no key and no value; ``gate`` "head" or "element": the heads' outputs are multiplied by sigmoid(W_g x)
("g": [num_heads, hidden] or [num_heads * v_dim, hidden]) before the output projection; W_g is stacked
under [Wq; Wk; Wv], so the gate comes out of the same product (a run that reads another's keys and
values stacks it under its Wq); ``sinks`` "zero": the same term with a fixed score of 0 and no tensor (one is
added to the denominator); ``qk_norm_weights`` False (with ``qk_norm``): the heads are divided by their root
mean square and multiplied by nothing; ``q_temp`` = (coef, every): the query at position p is multiplied by
1 + coef * ln(floor((p + 1) / every) + 1) after its norm; ``distance_slopes`` = x: slope_h * (p - j) is taken
off the scaled score of key j, with slope_h = 2^(-x (h + 1) / num_heads) for head h (a bias linear in the
distance, steeper for the first heads).

params: hidden_size, num_heads, num_kv_heads, head_dim, window (None: all
keys), scale (None: 1/sqrt(head_dim)), position (PartSpec), shares_kv (True:
the run reads another run's cache, has no k/v projections and writes nothing),
v_dim (None: head_dim), qk_norm (None, or eps), bias, softcap, chunk, keep_first, sinks, gate,
tensor_names (the names of the four projection weights below the part's prefix,
keys "q", "k", "v", "o", with qk_norm also "q_norm", "k_norm": the architecture
gives them, the part knows none).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import KVCacheView, Mixer, StepContext
from .linear import fused_residual_takes, linear
from .registry import build_part, register_part
from .spec import KVPagesNeed, PartSpec, TensorSpec


@register_part("mixer", "attention")
class PagedAttention(Mixer):
    @property
    def graph_safe(self) -> bool:
        """forward launches kernels only; so a decode step can be captured if the position part's ``apply`` can."""
        return bool(self.position.graph_safe)

    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.get()
        self.hidden = int(p["hidden_size"])
        self.nq = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.d = int(p["head_dim"])
        self.window = p.get("window")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.d)
        self.shares_kv = bool(p.get("shares_kv", False))
        self.dv = int(p.get("v_dim") or self.d)
        self.qk_eps = float(p["qk_norm"]) if p.get("qk_norm") is not None else None
        self.bias = bool(p.get("bias", False))
        self.softcap = float(p["softcap"]) if p.get("softcap") else 0.0
        self.chunk = int(p["chunk"]) if p.get("chunk") else 0
        self.keep_first = int(p.get("keep_first") or 0)
        self.sinks = bool(p.get("sinks", False))
        self.zero_sinks = p.get("sinks") == "zero"
        self.qk_weights = bool(p.get("qk_norm_weights", True))
        qt = p.get("q_temp")
        self.q_temp = (float(qt[0]), int(qt[1])) if qt else None
        if self.q_temp is not None and self.q_temp[1] < 1:
            raise ValueError("q_temp = (coef, every) with every >= 1")
        self.slope_exp = float(p["distance_slopes"]) if p.get("distance_slopes") is not None else None
        self.gate = p.get("gate")
        if self.gate not in (None, "head", "element"):
            raise ValueError(f"gate {self.gate!r}; known: None, 'head', 'element'")
        if self.keep_first and self.window is None:
            raise ValueError("keep_first goes with a window")
        if self.softcap < 0 or self.chunk < 0 or self.keep_first < 0:
            raise ValueError("softcap, chunk and keep_first must not be negative")
        # what the kernels of the Llama's form do not have: these go through the pages
        self.masked = bool(self.softcap or self.chunk or self.keep_first or self.sinks or self.gate or
                           self.q_temp or self.slope_exp is not None)
        # the Llama's form: rotation fused with the write
        self.plain = self.dv == self.d and self.qk_eps is None and not self.bias and not self.masked
        # keys and values of two sizes: where the larger one is a size of the tensor-core kernels, the pages keep
        # rows of that size for both (the rest zeros: no score changes, the result gains columns of zeros), and
        # those kernels serve; twice the pages' bytes for the smaller of the two against CUDA-core attention
        import os
        self.dp = max(self.d, self.dv)
        if self.d == self.dv or self.dp not in (16, 32, 64, 128) or self.nq // max(1, self.nkv) > 16 or \
                self.masked or os.environ.get("RLLM_ATTENTION_PAD") == "0":
            self.dp = 0
        if self.nq % self.nkv:
            raise ValueError(f"num_heads {self.nq} must be a multiple of num_kv_heads {self.nkv}")
        if self.plain and (self.d % 16 or self.d > 256):
            raise ValueError(f"head_dim {self.d}: the attention kernels take multiples of 16 up to 256")
        if self.dv > 256:
            raise ValueError(f"v_dim {self.dv}: the attention kernels take value heads up to 256")
        names = dict(p.get("tensor_names") or ())
        want = ["k", "o", "q", "v"] + (["k_norm", "q_norm"] if self.qk_eps is not None and self.qk_weights else []) + \
            (["q_bias", "k_bias", "v_bias", "o_bias"] if self.bias else []) + \
            (["sink"] if self.sinks and not self.zero_sinks else []) + (["g"] if self.gate else [])
        if sorted(names) != sorted(want):
            raise ValueError(f"an attention spec names its weights: tensor_names with the keys {sorted(want)}")
        self.names = {k: str(v) for k, v in names.items()}
        pos = p.get("position")
        self.position = build_part("position_encoding", pos if pos is not None else PartSpec.of("none"),
                                   prefix=prefix)
        if getattr(self.position, "interleaved", False):
            raise ValueError("this mixer's kernels rotate halves; an interleaved rotation is not among them")
        if not self.plain and self.position.fused_rotary() is None:
            raise ValueError("attention through the pages takes a rotation that its kernel can apply, or none")
        if self.shares_kv and self.bias:
            raise ValueError("a run that reads another's keys and values takes no biases")
        if not self.qk_weights and self.qk_eps is None:
            raise ValueError("qk_norm_weights False goes with qk_norm")
        self.gate_width = 0 if not self.gate else (self.nq if self.gate == "head" else self.nq * self.dv)
        self.w_qn = self.w_kn = None
        self.b_qkv = self.b_o = self.sink = self.slopes = None
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    # -- weights ----------------------------------------------------------
    def _names(self):
        p = self.prefix
        return tuple(p + self.names[k] for k in ("q", "k", "v", "o"))

    def ignored_tensors(self) -> List[str]:
        return self.position.ignored_tensors()

    def tensor_specs(self) -> List[TensorSpec]:
        q, k, v, o = self._names()
        specs = [TensorSpec(q, (self.nq * self.d, self.hidden))]
        if not self.shares_kv:
            specs += [TensorSpec(k, (self.nkv * self.d, self.hidden)),
                      TensorSpec(v, (self.nkv * self.dv, self.hidden))]
        specs.append(TensorSpec(o, (self.hidden, self.nq * self.dv)))
        if self.qk_eps is not None and self.qk_weights:
            specs.append(TensorSpec(self.prefix + self.names["q_norm"], (self.d,), role="vector",
                                    init=("one_plus_normal", 0.1)))
            if not self.shares_kv:
                specs.append(TensorSpec(self.prefix + self.names["k_norm"], (self.d,), role="vector",
                                        init=("one_plus_normal", 0.1)))
        if self.bias:
            for key, n in (("q_bias", self.nq * self.d), ("k_bias", self.nkv * self.d), ("v_bias", self.nkv * self.dv),
                           ("o_bias", self.hidden)):
                specs.append(TensorSpec(self.prefix + self.names[key], (n,), role="vector", init=("normal", 0.1)))
        if self.sinks and not self.zero_sinks:
            specs.append(TensorSpec(self.prefix + self.names["sink"], (self.nq,), role="vector", init=("normal", 1.0)))
        if self.gate:
            specs.append(TensorSpec(self.prefix + self.names["g"], (self.gate_width, self.hidden)))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        q, k, v, o = self._names()
        if self.shares_kv:
            # with a gate [Wq; Wg]: the gate's pre-activations lie behind the query heads
            stack = [tensors[q]] + ([tensors[self.prefix + self.names["g"]]] if self.gate else [])
            rows = sum(t.shape[0] for t in stack)
            if self.gate and rows % 8:
                stack.append(stack[0].new_zeros((8 - rows % 8, self.hidden)))
            self.w_qkv = torch.cat(stack, dim=0).contiguous() if self.gate else tensors[q]
        else:
            # stacked [Wq; Wk; Wv]: one matrix product gives a token's q, k and v side by side
            # (with a gate: [Wq; Wk; Wv; Wg], and the gate's pre-activations lie behind the value heads)
            stack = [tensors[q], tensors[k], tensors[v]] + ([tensors[self.prefix + self.names["g"]]] if self.gate else [])
            rows = sum(t.shape[0] for t in stack)
            if self.gate and rows % 8:
                # rows of zeros, so that a token's row of the product starts on a 16-byte boundary in bfloat16
                # (the tensor-core attention fetches its queries 16 bytes at a time)
                stack.append(stack[0].new_zeros((8 - rows % 8, self.hidden)))
            self.w_qkv = torch.cat(stack, dim=0).contiguous()
        self.w_o = tensors[o]
        if self.bias:
            # biases and sinks enter float32 arithmetic: kept so, whatever the run's dtype
            self.b_qkv = torch.cat([tensors[self.prefix + self.names[key]].float()
                                    for key in ("q_bias", "k_bias", "v_bias")]).contiguous()
            self.b_o = tensors[self.prefix + self.names["o_bias"]].float().contiguous()
        if self.zero_sinks:
            self.sink = torch.zeros(self.nq, dtype=torch.float32, device=self.w_o.device)
        elif self.sinks:
            self.sink = tensors[self.prefix + self.names["sink"]].float().contiguous()
        if self.slope_exp is not None:
            self.slopes = torch.tensor([2.0 ** (-self.slope_exp * (h + 1) / self.nq) for h in range(self.nq)],
                                       dtype=torch.float32, device=self.w_o.device)
        if self.dp and self.dv < self.dp:
            # the attention's result has dp columns a head, the last ones zeros: the projection skips them
            w = self.w_o.new_zeros((self.hidden, self.nq, self.dp))
            w[:, :, :self.dv] = self.w_o.view(self.hidden, self.nq, self.dv)
            self.w_o = w.view(self.hidden, self.nq * self.dp).contiguous()
        if self.qk_eps is not None and self.qk_weights:
            self.w_qn = tensors[self.prefix + self.names["q_norm"]].contiguous()
            self.w_kn = self.w_qn if self.shares_kv else \
                tensors[self.prefix + self.names["k_norm"]].to(self.w_qn.dtype).contiguous()

    def cache_need(self):
        if self.dp:
            return KVPagesNeed(self.nkv, self.dp, self.window)
        return KVPagesNeed(self.nkv, self.d, self.window, v_dim=None if self.dv == self.d else self.dv,
                           keep_first=self.keep_first, chunk=self.chunk or None)

    # -- compute ----------------------------------------------------------
    def fused_residual(self, num_rows: int, dtype: torch.dtype) -> bool:
        return self.plain and fused_residual_takes(num_rows, dtype, self.w_qkv, self.w_o)

    def _attend_from_pages(self, qkv: torch.Tensor, ctx: StepContext, cache: KVCacheView) -> torch.Tensor:
        """Heads with norms or values of their own size: one kernel normalises the queries in place and writes
        the (normalised) keys and the values into the pages; the attention then reads every key, the tokens'
        own included, from the pages.  Where keys and values have one size, the tensor-core kernels take it
        from there; else the CUDA-core kernel, which takes any two sizes."""
        T = qkv.shape[0]
        table = ctx.block_tables[cache.group]
        writes = cache.writes and not self.shares_kv
        q_pad = torch.empty((T, self.nq * self.dp), dtype=qkv.dtype, device=qkv.device) if self.dp else None
        inv_freq, rd = self.position.fused_rotary(qkv.device)
        mag = float(getattr(self.position, "magnitude", 1.0))
        # single decoded tokens of a mixer with options, where the tensor-core decode kernel serves: bias,
        # rotation and cache write ride in that kernel (the same arithmetic), and only the prompt portions'
        # rows are prepared here
        nd_fused = ctx.num_decode if (self.masked and self.qk_eps is None and not self.q_temp and writes and
                                      not self.dp and self.slopes is None and
                                      self.dv == self.d and self.d % 16 == 0 and
                                      ops.use_mma_attention(qkv.dtype, self.nq, self.nkv, self.d)) else 0
        if T > nd_fused:
            ops.head_norm_kv_write(qkv[nd_fused:], ctx.positions[nd_fused:], ctx.token_seq[nd_fused:], self.w_qn,
                                   self.w_kn, self.qk_eps or 0.0, table, cache.k, cache.v, self.nq,
                                   0 if self.shares_kv else self.nkv, self.d, self.dv, ctx.err, write_kv=writes,
                                   q_out=q_pad, bias=self.b_qkv, inv_freq=inv_freq, rotary_dim=rd, magnitude=mag,
                                   unit_norm=self.qk_eps is not None and not self.qk_weights, q_temp=self.q_temp)
        d, dv = (self.dp, self.dp) if self.dp else (self.d, self.dv)
        if q_pad is not None:
            qkv = q_pad
        out = torch.empty((T, self.nq * dv), dtype=qkv.dtype, device=qkv.device)
        window, stride = int(self.window or 0), qkv.shape[1]
        gate = None
        if self.gate:
            at = self.nq * self.d + (0 if self.shares_kv else self.nkv * (self.d + self.dv))
            gate = qkv[:, at: at + self.gate_width]
        opts = dict(keep_first=self.keep_first, chunk=self.chunk, softcap=self.softcap, sinks=self.sink, gate=gate,
                    gate_per_head=self.gate == "head") if self.masked else {}
        if self.slopes is not None:
            opts["slopes"] = self.slopes
        if dv == d and d % 16 == 0 and ops.use_mma_attention(qkv.dtype, self.nq, self.nkv, d):
            nd = ctx.num_decode
            if nd:
                fused = dict(inv_freq=inv_freq, rotary_dim=rd, write_kv=True, bias=self.b_qkv, magnitude=mag) \
                    if nd_fused else dict(write_kv=False)
                ops.attention_decode_bf16(qkv, stride, out, cache.k, cache.v, table, ctx.seq_lens, nd,
                                          max(ctx.seq_lens_host[:nd]), self.nq, self.nkv, d, window, self.scale,
                                          ctx.err, **fused, **opts)
            if T > nd:
                if ops.use_tcgen05_attention(qkv.dtype, self.nq, self.nkv, d, cache.k.shape[2]):
                    ops.attention_prefill_tcgen05(qkv, stride, out, cache.k, cache.v, table, ctx.q_start,
                                                  ctx.seq_lens, nd, ctx.num_seqs, T - nd, self.nq, self.nkv, d,
                                                  window, self.scale, ctx.err, **opts)
                else:
                    ops.attention_prefill_bf16(qkv, stride, out, cache.k, cache.v, table, ctx.q_start, ctx.seq_lens,
                                               nd, ctx.num_seqs, T - nd, self.nq, self.nkv, d, window,
                                               self.scale, ctx.err, **opts)
            return out
        ops.attention_simt_kv(qkv, stride, out, cache.k, cache.v, table, ctx.positions, ctx.token_seq, self.nq,
                              self.nkv, window, self.scale, ctx.err, **opts)
        return out

    def deferred_output_bias(self) -> Optional[torch.Tensor]:
        """The output projection's bias (float32 [hidden]) for a block that adds it where it completes the
        stream (it then calls ``forward`` with ``add_output_bias=False``); None: there is none."""
        return self.b_o

    def forward(self, x, ctx: StepContext, cache: KVCacheView, residual=None, add_output_bias: bool = True):
        out = self.attend(linear(x, self.w_qkv), ctx, cache)          # qkv [T, (nq + 2 nkv) d (+ the gate's)]
        y = linear(out, self.w_o, residual=residual)
        if self.b_o is not None and add_output_bias:
            ops.add_row_bias(y, self.b_o)
        return y

    def attend(self, qkv: torch.Tensor, ctx: StepContext, cache: KVCacheView) -> torch.Tensor:
        """From the tokens' projections (q, k and v heads side by side) to the attention's output
        [T, nq * d], before the output projection: position encoding, cache write, attention."""
        if not self.plain:
            return self._attend_from_pages(qkv, ctx, cache)
        x = qkv
        T = qkv.shape[0]
        nkv_here = 0 if self.shares_kv else self.nkv
        table = ctx.block_tables[cache.group]
        fused = self.position.fused_rotary(x.device)
        writes = cache.writes and not self.shares_kv
        if fused is None:
            q = qkv[:, : self.nq * self.d].view(T, self.nq, self.d)
            k = qkv[:, self.nq * self.d: (self.nq + nkv_here) * self.d].view(T, nkv_here, self.d) \
                if nkv_here else None
            self.position.apply(q, k, ctx.positions)
            fused = (None, 0)
        inv_freq, rd = fused
        out = torch.empty((T, self.nq * self.d), dtype=x.dtype, device=x.device)
        window = int(self.window or 0)
        stride = qkv.shape[1]
        use_mma = ops.use_mma_attention(x.dtype, self.nq, self.nkv, self.d)
        # sequences with one token: rotation, cache write and attention in one kernel
        nd = ctx.num_decode if use_mma else 0
        if nd:
            ops.attention_decode_bf16(qkv, stride, out, cache.k, cache.v, table, ctx.seq_lens, nd,
                                      max(ctx.seq_lens_host[:nd]), self.nq, self.nkv, self.d, window, self.scale,
                                      ctx.err, inv_freq=inv_freq, rotary_dim=rd, write_kv=writes)
        if T > nd:
            ops.rope_kv_write(qkv[nd:], ctx.positions[nd:], ctx.token_seq[nd:], inv_freq, rd, table, cache.k,
                              cache.v, self.nq, nkv_here, self.d, ctx.err, write_kv=writes)
            if ops.use_tcgen05_attention(x.dtype, self.nq, self.nkv, self.d, cache.k.shape[2]):
                ops.attention_prefill_tcgen05(qkv, stride, out, cache.k, cache.v, table, ctx.q_start, ctx.seq_lens,
                                              nd, ctx.num_seqs, T - nd, self.nq, self.nkv, self.d, window,
                                              self.scale, ctx.err)
            elif use_mma:
                ops.attention_prefill_bf16(qkv, stride, out, cache.k, cache.v, table, ctx.q_start, ctx.seq_lens,
                                           nd, ctx.num_seqs, T - nd, self.nq, self.nkv, self.d, window,
                                           self.scale, ctx.err)
            else:
                ops.attention_simt(qkv, stride, out, cache.k, cache.v, table, ctx.positions, ctx.token_seq,
                                   self.nq, self.nkv, self.d, window, self.scale, ctx.err)
        return out
