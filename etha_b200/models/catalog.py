"""Parameter shapes of decoder-only transformer families and the two layouts a weight sync bridges.

A weight sync moves every parameter from the trainer's layout (FSDP `Shard(0)`, HSDP, EP ...) into the
inference engine's tensor-parallel layout.  The reference's example derives the consumer placements
by walking vLLM modules (examples/vllm_weight_sync/vllm_server.py:87-126: column-parallel -> Shard(0),
row-parallel -> Shard(1), vocab-parallel embedding -> Shard(0), everything else Replicate); with no
network and no checkpoints here the same rules are applied to the shape catalog directly, and weights
are random-initialised.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

from torch.distributed.tensor.placement_types import Placement, Replicate, Shard


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: tuple[int, ...]
    kind: str  # "column" | "row" | "vocab" | "norm" | "expert_column" | "expert_row" | "router"


@dataclass
class ModelSpec:
    name: str
    tensors: list[TensorSpec] = field(default_factory=list)

    @property
    def numel(self) -> int:
        n = 0
        for t in self.tensors:
            k = 1
            for s in t.shape:
                k *= s
            n += k
        return n


def _decoder(name, layers, hidden, ffn, q_heads, kv_heads, head_dim, vocab, tied=False, experts=0, qk_norm=False) -> ModelSpec:
    m = ModelSpec(name)
    add = lambda n, shape, kind: m.tensors.append(TensorSpec(n, tuple(shape), kind))
    add("model.embed_tokens.weight", (vocab, hidden), "vocab")
    for i in range(layers):
        p = f"model.layers.{i}"
        add(f"{p}.input_layernorm.weight", (hidden,), "norm")
        add(f"{p}.self_attn.q_proj.weight", (q_heads * head_dim, hidden), "column")
        add(f"{p}.self_attn.k_proj.weight", (kv_heads * head_dim, hidden), "column")
        add(f"{p}.self_attn.v_proj.weight", (kv_heads * head_dim, hidden), "column")
        add(f"{p}.self_attn.o_proj.weight", (hidden, q_heads * head_dim), "row")
        if qk_norm:
            add(f"{p}.self_attn.q_norm.weight", (head_dim,), "norm")
            add(f"{p}.self_attn.k_norm.weight", (head_dim,), "norm")
        add(f"{p}.post_attention_layernorm.weight", (hidden,), "norm")
        if experts:
            add(f"{p}.block_sparse_moe.gate.weight", (experts, hidden), "router")
            add(f"{p}.block_sparse_moe.experts.w1", (experts, ffn, hidden), "expert_column")
            add(f"{p}.block_sparse_moe.experts.w3", (experts, ffn, hidden), "expert_column")
            add(f"{p}.block_sparse_moe.experts.w2", (experts, hidden, ffn), "expert_row")
        else:
            add(f"{p}.mlp.gate_proj.weight", (ffn, hidden), "column")
            add(f"{p}.mlp.up_proj.weight", (ffn, hidden), "column")
            add(f"{p}.mlp.down_proj.weight", (hidden, ffn), "row")
    add("model.norm.weight", (hidden,), "norm")
    if not tied:
        add("lm_head.weight", (vocab, hidden), "vocab")
    return m


def llama3_8b() -> ModelSpec:
    return _decoder("llama3-8b", 32, 4096, 14336, 32, 8, 128, 128256)


def qwen2_7b() -> ModelSpec:
    return _decoder("qwen2-7b", 28, 3584, 18944, 28, 4, 128, 152064)


def mixtral_8x7b() -> ModelSpec:
    return _decoder("mixtral-8x7b", 32, 4096, 14336, 32, 8, 128, 32000, experts=8)


def qwen3_0p6b() -> ModelSpec:
    return _decoder("qwen3-0.6b", 28, 1024, 3072, 16, 8, 128, 151936, tied=True, qk_norm=True)


def tiny_llama(layers: int = 2, hidden: int = 256, ffn: int = 512, vocab: int = 1024) -> ModelSpec:
    return _decoder("tiny-llama", layers, hidden, ffn, 4, 2, hidden // 4, vocab)


LayoutRule = Callable[[TensorSpec], tuple[Placement, ...]]


def fsdp_layout(mesh_ndim: int = 1, expert_parallel: bool = False) -> LayoutRule:
    """Trainer side: `Shard(0)` on the last mesh dim (earlier dims Replicate); with `expert_parallel`
    stacked expert weights are `Shard(0)` over experts, which is the same placement."""

    def rule(t: TensorSpec) -> tuple[Placement, ...]:
        return tuple([Replicate()] * (mesh_ndim - 1) + [Shard(0)])

    return rule


def vllm_tp_layout(mesh_ndim: int = 1) -> LayoutRule:
    """Inference side, tensor parallel over the last mesh dim."""

    def rule(t: TensorSpec) -> tuple[Placement, ...]:
        lead = [Replicate()] * (mesh_ndim - 1)
        if t.kind in ("column", "vocab"):
            last = Shard(0)
        elif t.kind == "row":
            last = Shard(1)
        elif t.kind == "expert_column":
            last = Shard(1)
        elif t.kind == "expert_row":
            last = Shard(2)
        else:
            last = Replicate()
        return tuple(lead + [last])

    return rule
