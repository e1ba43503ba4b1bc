"""Seeded synthetic workloads with the shapes of the benchmark configurations.

No checkpoint or dataset is involved: packed words are uniform random bits
(which is exactly uniform random codes at every width, including 3-bit),
scales are ``U(0.005, 0.02)`` in fp16 and offsets are the symmetric
``-2**(bits-1) * scale`` written out explicitly, as the format requires
(reference ``docs/format-spec.md:166-181``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .format import QuantTensor, row_geometry


def random_quant_tensor(
    rows: int,
    in_features: int,
    bits: int,
    *,
    group_size: int = 128,
    meta_dtype: torch.dtype = torch.float16,
    device: torch.device | str = "cpu",
    generator: torch.Generator | None = None,
) -> QuantTensor:
    """Uniform random codes with seeded fp16 scales; generated on ``device``."""
    g = row_geometry(bits, group_size, in_features)
    packed = torch.randint(
        -(2**31), 2**31, (rows, g.words_per_row), dtype=torch.int32, device=device, generator=generator
    )
    if g.is_per_row and (in_features * bits) % 32:
        # unused high bits of the last word must be zero
        keep = (1 << ((in_features * bits) % 32)) - 1
        packed[:, -1] &= keep
    scales = (torch.rand(rows, g.num_groups, device=device, generator=generator) * 0.015 + 0.005).to(meta_dtype)
    offsets = (-(1 << (bits - 1)) * scales.to(torch.float32)).to(meta_dtype)
    return QuantTensor(packed, scales, offsets, bits, g.group_size, in_features, (rows, in_features), symmetric=True)


@dataclass
class Module:
    name: str
    weight: QuantTensor
    input: str  # which activation buffer feeds it: "hidden" or "inter"


@dataclass
class LinearStack:
    """The packed linear modules one decode step of a dense transformer runs, in order."""

    name: str
    hidden: int
    intermediate: int
    modules: list[Module]
    bit_map: dict[str, int]

    @property
    def weight_bytes(self) -> int:
        return sum(m.weight.nbytes for m in self.modules)

    def stages(self) -> list[list[int]]:
        """Module indices grouped by data dependency, in execution order.

        Within a decoder layer q/k/v read the same hidden state, as do gate/up, so each of
        those sets is one stage whose members are independent; o_proj, down_proj and the
        lm_head are stages of their own.  Consecutive stages depend on each other.
        """
        out: list[list[int]] = []
        last_key = None
        for i, mod in enumerate(self.modules):
            leaf = mod.name.rsplit(".", 1)[-1]
            kind = {"q_proj": 0, "k_proj": 0, "v_proj": 0, "o_proj": 1, "gate_proj": 2, "up_proj": 2,
                    "down_proj": 3}.get(leaf, 4)
            key = (mod.name.split(".")[1] if mod.name.startswith("layers.") else mod.name, kind)
            if key != last_key:
                out.append([])
                last_key = key
            out[-1].append(i)
        return out

    def algorithmic_bytes(self, m: int, act_bytes: int = 2) -> int:
        """Weights (packed + scales + offsets) once, plus activations in and results out."""
        total = 0
        for mod in self.modules:
            qt = mod.weight
            total += qt.nbytes + m * qt.in_features * act_bytes + m * qt.num_rows * act_bytes
        return total


def seeded_bit_map(names: list[str], counts: dict[int, int], seed: int) -> dict[str, int]:
    """Assign widths to modules: a fixed multiset of widths, shuffled by ``seed``."""
    widths = [b for b, n in sorted(counts.items()) for _ in range(n)]
    if len(widths) != len(names):
        raise ValueError(f"{len(widths)} widths for {len(names)} modules")
    perm = torch.randperm(len(names), generator=torch.Generator().manual_seed(seed)).tolist()
    return {names[i]: widths[p] for i, p in enumerate(perm)}


def _decoder_layers(layers, hidden, inter, q_out, kv_out):
    shapes = [
        ("self_attn.q_proj", q_out, hidden, "hidden"),
        ("self_attn.k_proj", kv_out, hidden, "hidden"),
        ("self_attn.v_proj", kv_out, hidden, "hidden"),
        ("self_attn.o_proj", hidden, q_out, "attn"),
        ("mlp.gate_proj", inter, hidden, "hidden"),
        ("mlp.up_proj", inter, hidden, "hidden"),
        ("mlp.down_proj", hidden, inter, "inter"),
    ]
    return [(f"layers.{i}.{n}", r, k, src) for i in range(layers) for (n, r, k, src) in shapes]


def qwen2b_stack(device="cuda", seed: int = 20260, vocab: int = 248320, layers: int = 28) -> LinearStack:
    """28 layers, hidden 2048, intermediate 6144, 16 q / 8 kv heads of 128; 8-bit lm_head.

    Widths come from a seeded map over {2,3,4,8} whose nominal mean is 3.25 bits
    (54 / 79 / 53 / 10 modules of the 196).  ``vocab`` is 248,320, the shape of the
    reference benchmark's ``embed/lm_head`` row (``benchmarks/gemv_bandwidth.py:63``).
    """
    specs = _decoder_layers(layers, 2048, 6144, 16 * 128, 8 * 128)
    names = [s[0] for s in specs]
    if layers == 28:
        counts = {2: 54, 3: 79, 4: 53, 8: 10}
    else:  # reduced stacks (tests, profiling): same proportions, rounded
        n = len(names)
        c2, c3, c8 = round(n * 54 / 196), round(n * 79 / 196), max(1, round(n * 10 / 196))
        counts = {2: c2, 3: c3, 8: c8, 4: n - c2 - c3 - c8}
    bit_map = seeded_bit_map(names, counts, seed)
    gen = torch.Generator(device=device).manual_seed(seed)
    modules = [
        Module(n, random_quant_tensor(r, k, bit_map[n], device=device, generator=gen), src)
        for (n, r, k, src) in specs
    ]
    if vocab:
        bit_map["lm_head"] = 8
        modules.append(Module("lm_head", random_quant_tensor(vocab, 2048, 8, device=device, generator=gen), "hidden"))
    return LinearStack("qwen2b-3.25bit", 2048, 6144, modules, bit_map)


def qwen14b_linear_set(device="cuda", seed: int = 14014, layers: int = 40, shard: tuple[int, int] = (0, 1)) -> LinearStack:
    """40 layers, hidden 5120, intermediate 17408, 40 q / 8 kv heads; seeded 3/4-bit map.

    ``shard=(rank, world)`` keeps only this rank's contiguous slab of output rows
    of every module (column sharding).
    """
    rank, world = shard
    specs = _decoder_layers(layers, 5120, 17408, 40 * 128, 8 * 128)
    names = [s[0] for s in specs]
    n = len(names)
    bit_map = seeded_bit_map(names, {3: n // 2, 4: n - n // 2}, seed)
    gen = torch.Generator(device=device).manual_seed(seed + rank)
    modules = []
    for (name, r, k, src) in specs:
        if r % world:
            raise ValueError(f"{name}: {r} rows do not split over {world} ranks")
        modules.append(Module(name, random_quant_tensor(r // world, k, bit_map[name], device=device, generator=gen), src))
    return LinearStack(f"qwen3-14b-linear-set[{rank}/{world}]", 5120, 17408, modules, bit_map)


@dataclass
class MoeLayer:
    """One expert layer: the two packed banks plus seeded routing for ``tokens`` tokens."""

    hidden: int
    inter: int
    num_experts: int
    topk: int
    gate_up: QuantTensor  # [E * 2 * inter, hidden]
    down: QuantTensor  # [E * hidden, inter]

    def bytes_for(self, topk_ids: torch.Tensor, tokens: int, act_bytes: int = 2) -> int:
        """Algorithmic bytes of one step: every DISTINCT activated expert's packed rows once,
        plus token activations in and out and the routing table."""
        active = int(torch.unique(topk_ids[(topk_ids >= 0) & (topk_ids < self.num_experts)]).numel())
        per_expert = (self.gate_up.nbytes + self.down.nbytes) // self.num_experts
        return active * per_expert + tokens * self.hidden * act_bytes * 2 + tokens * self.topk * 8


def qwen3_moe_layer(device="cuda", seed: int = 3030, bits_gate_up: int = 3, bits_down: int = 4,
                    num_experts: int = 128, hidden: int = 2048, inter: int = 768, topk: int = 8) -> MoeLayer:
    """Qwen3-30B-A3B-shaped expert layer: 128 experts, top-8, hidden 2048, expert intermediate 768."""
    gen = torch.Generator(device=device).manual_seed(seed)
    gate_up = random_quant_tensor(num_experts * 2 * inter, hidden, bits_gate_up, device=device, generator=gen)
    down = random_quant_tensor(num_experts * hidden, inter, bits_down, device=device, generator=gen)
    return MoeLayer(hidden, inter, num_experts, topk, gate_up, down)


def seeded_routing(tokens: int, num_experts: int, topk: int, seed: int = 99, device="cpu"):
    """top-k of softmax(N(0,1) logits), weights renormalised over the selected experts."""
    gen = torch.Generator().manual_seed(seed)
    probs = torch.softmax(torch.randn(tokens, num_experts, generator=gen), dim=-1)
    w, ids = torch.topk(probs, topk, dim=-1)
    w = (w / w.sum(-1, keepdim=True)).to(torch.float32)
    return ids.to(torch.int32).to(device).contiguous(), w.to(device).contiguous()
