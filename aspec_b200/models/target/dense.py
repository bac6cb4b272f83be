"""In-framework Target: a frozen decoder-only LLM run prefill-only to produce Draft features.

The reference delegates the Target to SGLang and patches its models to capture hidden states
(aspec/inference/sglang_v0521.py:87-470, compat/patches/sglang-v0.5.21.patch:389-424); its semantic
reference is the hook-based HF wrapper aspec/models/target/eagle3_target_model.py:120-268.  Feature
contract reproduced here: for captured layer id ``k`` the feature is the residual-stream value *after*
decoder layer ``k`` (``hidden + residual`` as it enters layer ``k + 1``); ``last_hidden_states`` is the
post-final-norm hidden state; layout ``hidden_states [T, K * Dt]``.

Execution is packed (THD): one flat token array plus document lengths, causal attention restricted
to each document through the interval flash-attention kernel.  On CUDA every matrix product runs on
the framework's tcgen05 GEMM: q/k/v are one GEMM, gate/up one GEMM whose epilogue applies SwiGLU, and
the o_proj / down_proj GEMMs add the residual in their epilogue.  For a captured layer that epilogue
also writes the tile into the feature sink - which may be memory of the Draft GPUs (see
``transport.feature_ring``): capture costs no extra pass and no copy.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from aspec_b200.ops.attention import interval_attention_reference
from aspec_b200.ops.norm import rmsnorm_reference
from aspec_b200.ops.rope import RopeFrequencies, qk_norm_rope_reference


@dataclass
class TargetConfig:
    model_type: str = "qwen3"                 # qwen3 (q/k norm) | llama | ling_moe
    hidden_size: int = 4096
    intermediate_size: int = 12288
    num_hidden_layers: int = 36
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: Optional[int] = None
    vocab_size: int = 151936
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    max_position_embeddings: int = 40960
    qk_norm: Optional[bool] = None
    tie_word_embeddings: bool = False
    # MoE (ling_moe)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    num_shared_experts: int = 0
    moe_shared_expert_intermediate_size: int = 0
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    first_k_dense_replace: int = 0

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.qk_norm is None:
            self.qk_norm = self.model_type in ("qwen3", "ling_moe")

    @classmethod
    def from_file(cls, path: str) -> "TargetConfig":
        raw = json.load(open(path))
        raw = raw.get("text_config", raw)
        names = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in raw.items() if k in names})

    def to_dict(self) -> dict:
        return {k: getattr(self, k) for k in self.__dataclass_fields__}


class FeatureSink:
    """Where captured features go.  The default keeps them in local tensors."""

    def __init__(self, n_tokens: int, layer_ids: Sequence[int], hidden: int, device, dtype):
        self.layer_ids = list(layer_ids)
        self.hidden = hidden
        self.hidden_states = torch.empty(n_tokens, len(self.layer_ids) * hidden, device=device, dtype=dtype)
        self.last_hidden_states = torch.empty(n_tokens, hidden, device=device, dtype=dtype)

    def layer_views(self, layer_id: int) -> List[torch.Tensor]:
        """Destination views ``[T, Dt]`` (row stride ``K * Dt``) for one captured layer."""
        col = self.layer_ids.index(layer_id)
        return [self.hidden_states[:, col * self.hidden:(col + 1) * self.hidden]]

    def final_views(self) -> List[torch.Tensor]:
        return [self.last_hidden_states]


class _Layer(nn.Module):
    def __init__(self, cfg: TargetConfig, layer_idx: int, tp_rank: int = 0, tp_size: int = 1):
        super().__init__()
        d, D = cfg.head_dim, cfg.hidden_size
        # tensor parallel: this rank holds ``1 / tp_size`` of the heads and of the feed-forward width
        hq, hk = cfg.num_attention_heads // tp_size, cfg.num_key_value_heads // tp_size
        self.hq, self.hk = hq, hk
        self.cfg = cfg
        self.qkv_proj = nn.Parameter(torch.empty((hq + 2 * hk) * d, D))
        self.o_proj = nn.Parameter(torch.empty(D, hq * d))
        self.input_layernorm = nn.Parameter(torch.ones(D))
        self.post_attention_layernorm = nn.Parameter(torch.ones(D))
        if cfg.qk_norm:
            self.q_norm = nn.Parameter(torch.ones(d))
            self.k_norm = nn.Parameter(torch.ones(d))
        self.is_moe = cfg.num_experts > 0 and layer_idx >= cfg.first_k_dense_replace
        if self.is_moe:
            from aspec_b200.models.target.moe import TargetMoE
            self.mlp = TargetMoE(cfg, tp_rank, tp_size)
        else:
            self.gate_up_proj = nn.Parameter(torch.empty(2 * cfg.intermediate_size // tp_size, D))   # rows [gate | up]
            self.down_proj = nn.Parameter(torch.empty(D, cfg.intermediate_size // tp_size))
        self._gate_up_tiled = None


class DecodeCache:
    """Keys and values of ``sequences`` independent token sequences, ``capacity`` rows each, for every layer.

    One buffer per layer holds all sequences back to back (sequence ``r`` owns rows ``[r * capacity, (r + 1) *
    capacity)``), so that one attention launch serves all of them: a query names its own sequence's rows through its
    key interval, exactly as packed documents do in prefill."""

    def __init__(self, model: "DenseTarget", sequences: int, capacity: int):
        cfg = model.config
        dev, dtype = model.lm_head.device, model.lm_head.dtype
        self.sequences, self.capacity = int(sequences), int(capacity)
        shape = (self.sequences * self.capacity, model.layers[0].hk, cfg.head_dim)       # this rank's heads
        self.k = [torch.zeros(shape, device=dev, dtype=dtype) for _ in range(cfg.num_hidden_layers)]
        self.v = [torch.zeros(shape, device=dev, dtype=dtype) for _ in range(cfg.num_hidden_layers)]
        self.lengths = [0] * self.sequences
        # query positions per attention tile; ``None`` = ask the kernel wrapper (set by hand to exercise the padding on CPU)
        self.tile_positions: Optional[int] = None

    def accept(self, sequence: int, tokens: int) -> None:
        """Keep the first ``tokens`` rows that the last ``extend`` wrote for ``sequence``."""
        if tokens < 0 or self.lengths[sequence] + tokens > self.capacity:
            raise ValueError("accepted rows outside the cache")
        self.lengths[sequence] += int(tokens)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.k + self.v)


def tile_padding(counts: Sequence[int], per_tile: int, device):
    """Index maps that give every sequence query tiles of its own.

    The attention kernel walks, per query tile, the key tiles between the lowest and the highest key any row of the
    tile may see.  New tokens of different sequences point at cache regions that lie a whole ``capacity`` apart, so a
    tile shared by two sequences would walk everything between them.  Padding each sequence's rows to a multiple of the
    tile's ``per_tile`` positions (with repeats of its last row, dropped again afterwards) keeps each tile inside one
    sequence's region.  Returns ``(gather [Mp], keep [M])``: padded row -> source row, and where the real rows sit in the
    padded layout."""
    gather: List[int] = []
    keep: List[int] = []
    src = 0
    for m in counts:
        if m == 0:
            continue
        base = len(gather)
        gather += list(range(src, src + m)) + [src + m - 1] * (-m % per_tile)
        keep += list(range(base, base + m))
        src += m
    return (torch.tensor(gather, dtype=torch.long).to(device, non_blocking=True),
            torch.tensor(keep, dtype=torch.long).to(device, non_blocking=True))


class DenseTarget(nn.Module):
    """Qwen3 / Llama-shaped (optionally MoE) Target for prefill-only feature generation.

    ``tp_size > 1`` shards every layer over a group of ranks the way serving engines shard a model that does not fit one
    GPU (the reference passes ``target_tp_size`` to its serving engine, aspec/config/inference_config.py): attention
    heads and the feed-forward width are split (q/k/v and gate/up by output rows, o_proj and down_proj by input
    columns), experts of a mixture layer are dealt out whole, and the two partial sums per layer are all-reduced over
    ``tp_group``.  Embedding, norms and the output head stay whole on every rank, so every rank ends a pass with the
    same residual stream, features and logits."""

    def __init__(self, cfg: TargetConfig, tp_rank: int = 0, tp_size: int = 1, tp_group=None):
        super().__init__()
        self.config = cfg
        self.tp_rank, self.tp_size, self.tp_group = int(tp_rank), int(tp_size), tp_group
        if tp_size > 1:
            for what, n in (("num_attention_heads", cfg.num_attention_heads), ("num_key_value_heads", cfg.num_key_value_heads),
                            ("intermediate_size", cfg.intermediate_size if not cfg.num_experts or cfg.first_k_dense_replace else tp_size),
                            ("num_experts", cfg.num_experts or tp_size)):
                if n % tp_size:
                    raise ValueError(f"tensor parallel size {tp_size} must divide {what} ({n})")
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList([_Layer(cfg, i, self.tp_rank, self.tp_size) for i in range(cfg.num_hidden_layers)])
        self.norm = nn.Parameter(torch.ones(cfg.hidden_size))
        self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size))
        self.rope_freqs = RopeFrequencies(
            [cfg.rope_theta ** (-(2.0 * i) / cfg.head_dim) for i in range(cfg.head_dim // 2)])
        self.requires_grad_(False)

    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.02) -> "DenseTarget":
        # one generator per device, seeded here: the weights depend on ``seed`` alone, not on what else drew from the
        # global generator before (every Target replica of a run, and a Target built later to store features offline, are
        # the same model); generated on the parameter's device, so host memory stays flat
        gens = {}
        for name, p in self.named_parameters():
            if p.dim() >= 2:
                g = gens.get(p.device)
                if g is None:
                    g = gens[p.device] = torch.Generator(device=p.device)
                    g.manual_seed(int(seed))
                if self.tp_size == 1:
                    p.normal_(0.0, std, generator=g)
                else:
                    # draw the WHOLE tensor (one at a time) and keep this rank's part: the sharded model is the unsharded
                    # model of the same seed, whatever the group size
                    whole = torch.empty(self.whole_shape(name, p), device=p.device, dtype=p.dtype).normal_(0.0, std, generator=g)
                    p.copy_(self.shard_of(name, whole))
        return self

    # -- tensor-parallel layout ---------------------------------------------------------------------
    def whole_shape(self, name: str, p: torch.Tensor) -> tuple:
        """Shape of parameter ``name`` in the unsharded model."""
        t, leaf = self.tp_size, name.rsplit(".", 1)[-1]
        if t == 1 or not name.startswith("layers."):
            return tuple(p.shape)
        if leaf in ("qkv_proj", "gate_up_proj", "shared_gate_up") and p.dim() == 2:
            return (p.shape[0] * t, p.shape[1])
        if leaf in ("o_proj", "down_proj", "shared_down") and p.dim() == 2:
            return (p.shape[0], p.shape[1] * t)
        if leaf in ("gate_up_proj", "down_proj") and p.dim() == 3:          # expert banks: experts are dealt out whole
            return (p.shape[0] * t, *p.shape[1:])
        return tuple(p.shape)

    def shard_of(self, name: str, whole: torch.Tensor) -> torch.Tensor:
        """This rank's part of an unsharded parameter (a checkpoint tensor, or a freshly drawn one)."""
        t, r, leaf = self.tp_size, self.tp_rank, name.rsplit(".", 1)[-1]
        if t == 1 or not name.startswith("layers."):
            return whole
        part = lambda x, dim: x.chunk(t, dim)[r]
        if leaf == "qkv_proj":
            d, cfg = self.config.head_dim, self.config
            q, k, v = whole.split([cfg.num_attention_heads * d, cfg.num_key_value_heads * d, cfg.num_key_value_heads * d], 0)
            return torch.cat([part(q, 0), part(k, 0), part(v, 0)], 0)
        if leaf in ("gate_up_proj", "shared_gate_up") and whole.dim() == 2:
            gate, up = whole.chunk(2, 0)
            return torch.cat([part(gate, 0), part(up, 0)], 0)
        if leaf in ("o_proj", "down_proj", "shared_down") and whole.dim() == 2:
            return part(whole, 1)
        if leaf in ("gate_up_proj", "down_proj") and whole.dim() == 3:
            return part(whole, 0)
        return whole

    @torch.no_grad()
    def load_whole_state_dict(self, state: Dict[str, torch.Tensor]) -> None:
        """Load an unsharded checkpoint: every rank keeps its part of each tensor."""
        own = dict(self.named_parameters())
        own.update(dict(self.named_buffers()))
        missing = sorted(set(own) - set(state))
        if missing:
            raise KeyError(f"checkpoint lacks {missing[:4]}")
        for name, p in own.items():
            p.copy_(self.shard_of(name, state[name]).to(p.device, p.dtype))

    def _reduce(self, partial: torch.Tensor) -> torch.Tensor:
        if self.tp_size > 1:
            import torch.distributed as dist
            dist.all_reduce(partial, group=self.tp_group)
        return partial

    def agree(self, values: torch.Tensor) -> torch.Tensor:
        """Rank 0's values on every rank of the group: decisions taken from (equal, but separately computed) logits."""
        if self.tp_size > 1:
            import torch.distributed as dist
            values = values.contiguous()
            dist.broadcast(values, src=dist.get_global_rank(self.tp_group, 0) if self.tp_group is not None else 0, group=self.tp_group)
        return values

    # -- pieces ---------------------------------------------------------------------------------
    def _use_kernels(self, x: torch.Tensor) -> bool:
        return x.is_cuda and x.dtype == torch.bfloat16 and self.config.head_dim == 128

    def _tiled_gate_up(self, layer: _Layer) -> torch.Tensor:
        """gate/up rows interleaved in blocks of 128 so one GEMM tile holds matching gate and up columns."""
        if layer._gate_up_tiled is None:
            w = layer.gate_up_proj
            I = w.shape[0] // 2
            if I % 128:
                return None
            layer._gate_up_tiled = torch.stack([w[:I].view(I // 128, 128, -1), w[I:].view(I // 128, 128, -1)], 1) \
                .reshape(2 * I, -1).contiguous()
        return layer._gate_up_tiled

    def _attention(self, layer: _Layer, x, positions, intervals, kv=None):
        cfg = self.config
        hq, hk, d = layer.hq, layer.hk, cfg.head_dim
        T = x.shape[0]
        inv_freq = self.rope_freqs.get(x.device)
        if self._use_kernels(x):
            from aspec_b200.ops import attention_sm100 as A
            from aspec_b200.ops import elementwise_sm100 as E
            from aspec_b200.ops import gemm as G
            qkv = G.gemm(x, layer.qkv_proj)
            q = qkv[:, : hq * d].reshape(T, hq, d)
            k = qkv[:, hq * d:(hq + hk) * d].reshape(T, hk, d)
            v = qkv[:, (hq + hk) * d:].view(T, hk, d)
            qn = layer.q_norm if cfg.qk_norm else None
            kn = layer.k_norm if cfg.qk_norm else None
            q, _ = E.qk_norm_rope_fwd(q.contiguous(), qn, positions, inv_freq, cfg.rms_norm_eps, 1.0)
            k, _ = E.qk_norm_rope_fwd(k.contiguous(), kn, positions, inv_freq, cfg.rms_norm_eps, 1.0)
            if kv is not None:          # decode: the new rows join the cached keys / values and attend all of them
                k, v = kv[0].index_copy_(0, kv[2], k), kv[1].index_copy_(0, kv[2], v)
                if kv[3] is not None:   # one sequence per query tile (see ``tile_padding``)
                    o, _ = A.forward(q.index_select(0, kv[3][0]), k, v, intervals.index_select(0, kv[3][0]), d ** -0.5)
                    return o.index_select(0, kv[3][1]).view(T, hq * d)
            o, _ = A.forward(q, k, v, intervals, d ** -0.5)
            return o.view(T, hq * d)
        qkv = F.linear(x, layer.qkv_proj)
        q = qkv[:, : hq * d].reshape(T, hq, d)
        k = qkv[:, hq * d:(hq + hk) * d].reshape(T, hk, d)
        v = qkv[:, (hq + hk) * d:].reshape(T, hk, d)
        q = qk_norm_rope_reference(q, layer.q_norm if cfg.qk_norm else None, positions, inv_freq, cfg.rms_norm_eps)
        k = qk_norm_rope_reference(k, layer.k_norm if cfg.qk_norm else None, positions, inv_freq, cfg.rms_norm_eps)
        if kv is not None:
            k, v = kv[0].index_copy_(0, kv[2], k.to(kv[0].dtype)), kv[1].index_copy_(0, kv[2], v.to(kv[1].dtype))
            if kv[3] is not None:
                o, _ = interval_attention_reference(q.index_select(0, kv[3][0]), k, v, intervals.index_select(0, kv[3][0]), d ** -0.5)
                return o.index_select(0, kv[3][1]).reshape(T, hq * d)
        o, _ = interval_attention_reference(q, k, v, intervals, d ** -0.5)
        return o.reshape(T, hq * d)

    def _logits(self, final):
        if self._use_kernels(final) and self.lm_head.shape[0] % 8 == 0:
            from aspec_b200.ops import gemm as G
            return G.gemm(final, self.lm_head)
        return F.linear(final, self.lm_head)

    def _norm(self, x, w, out=None):
        if self._use_kernels(x):
            from aspec_b200.ops import elementwise_sm100 as E
            y, _ = E.rmsnorm_fwd(x, w, self.config.rms_norm_eps)
            return y
        return rmsnorm_reference(x, w, self.config.rms_norm_eps)

    def _proj_residual(self, a, w, residual, mirrors=None):
        """``residual + a @ w.T`` with the add (and the optional mirrored stores) in the GEMM epilogue.

        ``mirrors`` is a list of destination views of the whole output, or a list of ``(row_start, row_end, views)``
        segments when several requests were batched into one prefill: then the product runs once per segment so that
        each request's rows go to its own destinations."""
        if self.tp_size > 1:
            # partial product of this rank's columns, summed over the group, then the residual and the feature stores
            if self._use_kernels(a):
                from aspec_b200.ops import gemm as G
                part = G.gemm(a, w)
            else:
                part = F.linear(a, w)
            return self._finish_reduced(self._reduce(part), residual, mirrors)
        if mirrors and isinstance(mirrors[0], tuple):
            out = torch.empty_like(residual)
            for r0, r1, views in mirrors:
                out[r0:r1] = self._proj_residual(a[r0:r1], w, residual[r0:r1], views)
            return out
        if self._use_kernels(a):
            from aspec_b200.ops import gemm as G
            return G.gemm(a, w, addend=residual, mirrors=mirrors or None)
        out = residual + F.linear(a, w)
        for m in mirrors or ():
            m.copy_(out)
        return out

    @staticmethod
    def _finish_reduced(reduced, residual, mirrors):
        out = residual + reduced
        for m in mirrors or ():
            if isinstance(m, tuple):
                for view in m[2]:
                    view.copy_(out[m[0]:m[1]])
            else:
                m.copy_(out)
        return out

    def _mlp(self, layer: _Layer, x, residual, mirrors):
        if layer.is_moe:
            return self._finish_reduced(self._reduce(layer.mlp(x)), residual, mirrors)
        if self._use_kernels(x):
            from aspec_b200.ops import gemm as G
            tiled = self._tiled_gate_up(layer)
            if tiled is not None:
                act = G.gemm(x, tiled, epilogue=G.EPI_SWIGLU)
            else:
                from aspec_b200.ops.activation import swiglu
                act = swiglu(G.gemm(x, layer.gate_up_proj))
            return self._proj_residual(act, layer.down_proj, residual, mirrors)
        gu = F.linear(x, layer.gate_up_proj)
        g, u = gu.chunk(2, -1)
        return self._proj_residual(F.silu(g) * u, layer.down_proj, residual, mirrors)

    # -- prefill ----------------------------------------------------------------------------------
    @staticmethod
    def causal_intervals(document_lengths: Sequence[int], device) -> torch.Tensor:
        """Interval table of packed causal attention: token ``i`` sees ``[doc_start, i + 1)``."""
        starts = torch.repeat_interleave(
            torch.tensor([0] + list(torch.tensor(document_lengths).cumsum(0)[:-1].tolist())),
            torch.tensor(document_lengths))
        T = int(sum(document_lengths))
        iv = torch.zeros(T, 4, dtype=torch.int32)
        iv[:, 0] = starts.to(torch.int32)
        iv[:, 1] = torch.arange(1, T + 1, dtype=torch.int32)
        return iv.to(device, non_blocking=True)

    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, document_lengths: Sequence[int], capture_layers: Sequence[int],
                sink=None, want_logits: bool = False) -> Dict[str, torch.Tensor]:
        """``input_ids [T]`` (packed documents).  Returns the sink's tensors (and logits when asked).

        ``sink`` may be a list of ``(row_start, row_end, sink)`` segments: several requests batched into one pass (larger
        GEMMs), each with its own destinations."""
        cfg = self.config
        T = input_ids.shape[0]
        dev = input_ids.device
        if sum(document_lengths) != T:
            raise ValueError("document_lengths must sum to the number of tokens")
        x = self.embed_tokens(input_ids)
        segments = sink if isinstance(sink, list) else None
        if sink is None:
            sink = FeatureSink(T, capture_layers, cfg.hidden_size, dev, x.dtype)
        pos_list = torch.cat([torch.arange(n) for n in document_lengths]).to(torch.int32)
        positions = pos_list.to(dev, non_blocking=True)
        intervals = self.causal_intervals(document_lengths, dev)
        capture = set(capture_layers)
        for i, layer in enumerate(self.layers):
            h = self._norm(x, layer.input_layernorm)
            a = self._attention(layer, h, positions, intervals)
            x = self._proj_residual(a, layer.o_proj, x)
            h = self._norm(x, layer.post_attention_layernorm)
            if i not in capture:
                mirrors = None
            elif segments is not None:
                mirrors = [(r0, r1, sk.layer_views(i)) for r0, r1, sk in segments]
            else:
                mirrors = sink.layer_views(i)
            x = self._mlp(layer, h, x, mirrors)
        final = self._norm(x, self.norm)
        if segments is not None:
            for r0, r1, sk in segments:
                for view in sk.final_views():
                    view.copy_(final[r0:r1])
            return {"final_hidden": final}
        for view in sink.final_views():
            view.copy_(final)
        out = {"hidden_states": getattr(sink, "hidden_states", None),
               "last_hidden_states": getattr(sink, "last_hidden_states", None), "final_hidden": final}
        if want_logits:
            out["logits"] = self._logits(final)
        return out

    # -- decode with cached keys / values ------------------------------------------------------------
    def new_decode_cache(self, sequences: int, capacity: int) -> "DecodeCache":
        return DecodeCache(self, sequences, capacity)

    @torch.no_grad()
    def extend(self, cache: "DecodeCache", new_ids: Sequence[torch.Tensor], capture_layers: Sequence[int] = ()) -> Dict[str, torch.Tensor]:
        """One pass over the NEW tokens of several sequences at once (``new_ids[r]``: the tokens of sequence ``r`` that
        the cache does not hold yet; empty for a sequence that sits this pass out).  Token ``j`` of sequence ``r`` takes
        position ``cache.lengths[r] + j`` and attends the cached rows of its own sequence plus the new tokens up to
        itself.  The new keys / values are written behind each sequence's cached rows but the lengths do not move: the
        caller keeps what it accepts with ``cache.accept(r, n)`` and the rest is overwritten by the next pass - which is
        what speculative verification needs (reference: the serving engine's decode and verify passes,
        aspec/inference/engine/sgl_engine_decode.py:39-424).

        Returns ``logits [M, V]``, ``hidden_states [M, K * D]`` of the captured layers and ``offsets`` (where each
        sequence's rows start in those), ``M`` = all new tokens."""
        cfg = self.config
        dev = self.lm_head.device
        counts = [int(t.numel()) for t in new_ids]
        if len(counts) != cache.sequences:
            raise ValueError("one (possibly empty) tensor of new tokens per cached sequence")
        for r, m in enumerate(counts):
            if cache.lengths[r] + m > cache.capacity:
                raise ValueError(f"sequence {r}: {cache.lengths[r]} cached + {m} new tokens exceed the cache's {cache.capacity}")
        M = sum(counts)
        if M == 0:
            raise ValueError("no new tokens")
        pos = torch.cat([torch.arange(cache.lengths[r], cache.lengths[r] + m) for r, m in enumerate(counts)])
        base = torch.cat([torch.full((m,), r * cache.capacity) for r, m in enumerate(counts)])
        iv = torch.zeros(M, 4, dtype=torch.int32)
        iv[:, 0] = base.to(torch.int32)
        iv[:, 1] = (base + pos + 1).to(torch.int32)
        rows = (base + pos).to(dev, non_blocking=True)
        positions = pos.to(torch.int32).to(dev, non_blocking=True)
        intervals = iv.to(dev, non_blocking=True)
        x = self.embed_tokens(torch.cat([t.reshape(-1) for t in new_ids]).to(dev))
        per_tile = cache.tile_positions
        if per_tile is None and self._use_kernels(x):
            from aspec_b200.ops.attention_sm100 import positions_per_tile
            per_tile = positions_per_tile(self.layers[0].hq, self.layers[0].hk)
        padding = tile_padding(counts, per_tile, dev) if per_tile and sum(m > 0 for m in counts) > 1 else None
        sink = FeatureSink(M, capture_layers, cfg.hidden_size, dev, x.dtype)
        capture = set(capture_layers)
        for i, layer in enumerate(self.layers):
            h = self._norm(x, layer.input_layernorm)
            a = self._attention(layer, h, positions, intervals, kv=(cache.k[i], cache.v[i], rows, padding))
            x = self._proj_residual(a, layer.o_proj, x)
            h = self._norm(x, layer.post_attention_layernorm)
            x = self._mlp(layer, h, x, sink.layer_views(i) if i in capture else None)
        final = self._norm(x, self.norm)
        offsets = [0]
        for m in counts:
            offsets.append(offsets[-1] + m)
        return {"logits": self._logits(final), "hidden_states": sink.hidden_states, "offsets": offsets}

    def memory_bytes(self) -> int:
        return sum(p.numel() * p.element_size() for p in self.parameters())
