"""The step's forward pass launched from C++ where the model allows it.

The parts of a model stay what they are: declarative objects that own parameters and know how to
run themselves one kernel at a time (``parts/*.py``) -- that path takes any arrangement of parts,
the toy ones of the tests included.  But a step of the standard arrangement (every call site a
pre-norm block of RMSNorm -> paged attention with a whole-head rotate-half rotary encoding ->
RMSNorm -> SiLU-gated feed-forward; an embedding table in front, an RMSNorm and an output head
behind; one storage dtype throughout) is always the same sequence of launches, and walking it in
Python costs more host time than a prefill step's kernels take.  ``NativeForward.plan`` looks at the
parts the builder chose (their exact classes and sizes) and, if they are that arrangement, hands the
loop to ``csrc/cuda/step_forward.cu``: the same launchers in the same order, chosen by the same
rules, without an interpreter in between.  Anything else, and any step with forcing options
(``gemm``, ``attention``, ``attn_version``, ...), runs part by part.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..kernels import library as K
from ..parts.attention import PagedAttention
from ..parts.base import StepContext
from ..parts.block import PreNormBlock
from ..parts.embedding import Embedding, LMHead
from ..parts.mlp import GatedMLP
from ..parts.norm import RMSNorm
from ..parts.rope import RotaryEmbedding

LIBRARY_WORKSPACE_BYTES = 32 << 20
FORCING_OPTIONS = ("attention", "attn_version", "attn_parts", "attn_merge", "attn_prefill", "fuse")


def _same(dtype, *tensors) -> bool:
    return all(t is not None and t.dtype == dtype and t.is_contiguous() for t in tensors)


class NativeForward:
    def __init__(self, spec, runner, sizes: dict, layers, inv_freq: torch.Tensor, scale: float) -> None:
        self.spec, self.runner = spec, runner
        self.H, self.I, self.nh, self.nkv, self.hd = (sizes[k] for k in ("H", "I", "nh", "nkv", "hd"))
        self.vocab = spec.lm_head.vocab
        self.layers, self.inv_freq, self.scale = layers, inv_freq, scale        # `layers`: ctypes array, kept alive
        self.f32 = runner.dtype == torch.float32
        dev = runner.device
        self.sms = K.sm_count(dev)
        self.lib_workspace = None if self.f32 else torch.empty(LIBRARY_WORKSPACE_BYTES, dtype=torch.uint8, device=dev)
        # scratch of split-context decode attention beyond what one cluster merges: sized for the
        # engine's limits (requests x heads x partitions x (head_dim + 2) floats, 64 partitions)
        self.attn_scratch = None if self.f32 else torch.empty(
            min(runner.max_seqs, 1024) * self.nh * 64 * (self.hd + 2), dtype=torch.float32, device=dev)
        # partial sums of squares of the residual, one per 16 columns and row (None = norms are launches)
        fuse = runner.options.get("fuse_norms", True) and not self.f32
        self.norm_partials = torch.zeros((self.H + 15) // 16 * 16, dtype=torch.float32, device=dev) if fuse else None
        # cosines and sines of a step's angles, computed once a step for all layers (steps of many rows)
        self.rope_table = None if self.f32 else torch.empty(runner.max_rows * self.hd, dtype=torch.float32, device=dev)
        self.calls = 0

    # ------------------------------------------------------------------ does the model fit
    @classmethod
    def plan(cls, spec, runner) -> Optional["NativeForward"]:
        dtype = runner.dtype
        if dtype not in (torch.bfloat16, torch.float32) or runner.plan.has_state or not spec.order:
            return None
        if len(runner.plan.groups) > K.FORWARD_MAX_GROUPS or not K.forward_layouts_match():
            return None
        emb, fin, head = spec.embedding, spec.final_norm, spec.lm_head
        if type(emb) is not Embedding or type(fin) is not RMSNorm or type(head) is not LMHead:
            return None
        if not _same(dtype, emb.param("weight"), fin.param("weight"), head.param("weight")):
            return None
        sizes, inv_freq, scale = None, None, None
        layers = (K.ForwardLayer * len(spec.order))()
        for k, call in enumerate(spec.order):
            b = spec.blocks[call.layer]
            if type(b) is not PreNormBlock:
                return None
            n1, mx, n2, ff = b.norm1, b.mixer, b.norm2, b.ffn
            if type(n1) is not RMSNorm or type(n2) is not RMSNorm or type(mx) is not PagedAttention \
                    or type(ff) is not GatedMLP or type(mx.position) is not RotaryEmbedding:
                return None
            pos = mx.position
            if pos.interleaved or pos.rotary_dim != mx.hd or pos.inv_freq is None:
                return None
            t = (n1.param("weight"), n2.param("weight"), mx.qkv.param("weight"), mx.o.param("weight"),
                 ff.gate_up.param("weight"), ff.down.param("weight"))
            if not _same(dtype, *t):
                return None
            here = dict(H=mx.hidden, I=ff.intermediate, nh=mx.nh, nkv=mx.nkv, hd=mx.hd)
            if sizes is None:
                sizes, inv_freq, scale = here, pos.inv_freq, mx.scale
            elif here != sizes or mx.scale != scale or not torch.equal(pos.inv_freq, inv_freq):
                return None
            if ff.hidden != sizes["H"] or emb.hidden != sizes["H"] or head.hidden != sizes["H"]:
                return None
            site = runner.pools.sites[k]
            if site.k is None or site.state is not None or not _same(dtype, site.k, site.v):
                return None
            L = layers[k]
            L.norm1, L.norm2, L.w_qkv, L.w_o, L.w_gate_up, L.w_down = (x.data_ptr() for x in t)
            L.k_cache, L.v_cache = site.k.data_ptr(), site.v.data_ptr()
            L.eps1, L.eps2 = n1.eps, n2.eps
            L.group, L.window, L.writes, L.num_pages = site.group, mx.window, int(site.writes), site.k.shape[0]
        if dtype == torch.bfloat16 and (sizes["H"] % 8 or sizes["I"] % 8 or (sizes["nh"] * sizes["hd"]) % 8):
            return None                             # rows of the buffers must stay 16-byte aligned
        return cls(spec, runner, sizes, layers, inv_freq, scale)

    def model_for_core(self) -> dict:
        """The model as the C++ request loop wants it (csrc/core/native_engine.h: NativeModel)."""
        names = ("w_qkv", "w_o", "w_gate_up", "w_down", "norm1", "norm2", "k_cache", "v_cache")
        layers = []
        for L in self.layers:
            d = {k: int(getattr(L, k) or 0) for k in names}
            d.update(eps1=float(L.eps1), eps2=float(L.eps2), group=int(L.group), window=int(L.window),
                     writes=int(L.writes), num_pages=int(L.num_pages))
            layers.append(d)
        return dict(embed=self.spec.embedding.param("weight").data_ptr(),
                    final_norm=self.spec.final_norm.param("weight").data_ptr(),
                    lm_head=self.spec.lm_head.param("weight").data_ptr(), inv_freq=self.inv_freq.data_ptr(),
                    f32=int(self.f32), H=self.H, I=self.I, nh=self.nh, nkv=self.nkv, hd=self.hd, V=self.vocab,
                    sm_count=self.sms, final_eps=float(self.spec.final_norm.eps), scale=float(self.scale), layers=layers)

    # ------------------------------------------------------------------------- one step
    def takes(self, ctx: StepContext) -> bool:
        o = ctx.options
        return (o.get("native_forward", True) and o.get("gemm", "auto") == "auto"
                and not any(k in o for k in FORCING_OPTIONS) and ctx.tile_rows == 64)

    def run(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """Float32 logits [wanted rows, vocab] (None when no row is wanted).  Only enqueues device work."""
        T, n = ctx.rows, ctx.logit_rows.numel()
        dev, dt = self.runner.device, self.runner.dtype
        H, I, QK = self.H, self.I, self.nh * self.hd
        QKV = (self.nh + 2 * self.nkv) * self.hd

        def buf(rows, cols, dtype=dt):
            return torch.empty((rows, cols), dtype=dtype, device=dev)

        x, h, proj = buf(T, H, torch.float32), buf(T, H), buf(T, H)
        qkv, attn, act = buf(T, QKV), buf(T, QK), buf(T, I)
        fused_ff = (not self.f32) and K.gate_up_silu_supported(T, I, H)
        gate_up = None if fused_ff else buf(T, 2 * I)
        h_last = buf(n, H) if n else None
        logits = buf(n, self.vocab, torch.float32) if n else None
        a = K.ForwardArgs()
        a.layers = ctypes.addressof(self.layers)
        a.embed = self.spec.embedding.param("weight").data_ptr()
        a.final_norm = self.spec.final_norm.param("weight").data_ptr()
        a.lm_head = self.spec.lm_head.param("weight").data_ptr()
        a.inv_freq = self.inv_freq.data_ptr()
        a.tokens, a.positions, a.row_seq = ctx.tokens.data_ptr(), ctx.positions.data_ptr(), ctx.row_seq.data_ptr()
        a.seq_q_start, a.seq_q_len = ctx.seq_q_start.data_ptr(), ctx.seq_q_len.data_ptr()
        a.seq_ctx_len = ctx.seq_ctx_len.data_ptr()
        a.tile_seq, a.tile_q0 = ctx.tile_seq.data_ptr(), ctx.tile_q0.data_ptr()
        a.logit_rows = ctx.logit_rows.data_ptr()
        for g, view in enumerate(ctx.groups):
            a.group_tables[g] = view.block_tables.data_ptr()
            a.group_slots[g] = view.slot_mapping.data_ptr()
        a.x, a.h, a.qkv, a.attn, a.proj, a.act = (t.data_ptr() for t in (x, h, qkv, attn, proj, act))
        a.gate_up = gate_up.data_ptr() if gate_up is not None else None
        a.h_last = h_last.data_ptr() if n else None
        a.logits = logits.data_ptr() if n else None
        if self.attn_scratch is not None:
            a.attn_scratch, a.attn_scratch_floats = self.attn_scratch.data_ptr(), self.attn_scratch.numel()
        if self.lib_workspace is not None:
            a.lib_workspace, a.lib_workspace_bytes = self.lib_workspace.data_ptr(), self.lib_workspace.numel()
        if self.rope_table is not None:
            a.rope_table, a.rope_table_floats = self.rope_table.data_ptr(), self.rope_table.numel()
        if self.norm_partials is not None:
            a.norm_partials, a.norm_partials_floats = self.norm_partials.data_ptr(), self.norm_partials.numel()
        a.num_layers, a.f32 = len(self.layers), int(self.f32)
        a.H, a.I, a.nh, a.nkv, a.hd, a.V = H, I, self.nh, self.nkv, self.hd, self.vocab
        a.block_size, a.max_blocks = ctx.groups[0].block_size, ctx.groups[0].block_tables.shape[1]
        a.sm_count = self.sms
        a.rows, a.seqs, a.decode_seqs = T, ctx.seqs, ctx.decode_seqs
        a.prefill_tiles, a.tile_rows, a.max_decode_ctx, a.num_logits = ctx.prefill_tiles, ctx.tile_rows, ctx.max_decode_ctx, n
        a.final_eps, a.scale = self.spec.final_norm.eps, self.scale
        K.forward(a)
        self.calls += 1
        return logits
