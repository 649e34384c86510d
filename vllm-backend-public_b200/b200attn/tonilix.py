"""Tonilix decoder on the b200attn ops: pre-norm layers around one fp32 residual, the norm an RMS norm in groups, every
sublayer output scaled per channel before the residual sum, and the mixer's input blended per channel with the previous
token's normalised row (token shift; the previous row is per-sequence state).  The embedding adds sinusoidal positions
and is normalised.  A layer's sequence mixer is one of

* `channel_delta`: a gated delta-rule recurrence behind short causal convolutions whose decay acts per key channel
  (low-rank decay and output-gate projections, sigmoid output gate);
* `parallel`: two mixers that read the same input, summed with fixed weights -- softmax attention over paged K/V with
  biased projections, a query factor that grows with the logarithm of the position in steps, and a sigmoid output gate;
  and gated linear attention (decay per key channel = sigmoid^(1/tau) of a low-rank projection, RMS norm per head, SiLU
  gate).

The feed-forward is dense (gelu_tanh(gate) * up) or a routed mixture of ungated squared-ReLU experts whose router scores
are sigmoids, chosen with a correction inside the best groups of neighbouring experts, weights normalised and scaled.

The model plugs into the same engine as the other families (b200attn.engine.LLMEngine): paged K/V pools addressed through
the scheduler's block tables and slot mapping, recurrent state (matrix states, convolution tails, token-shift rows) in
the scheduler's per-sequence state slots, one forward over [decode rows | prompt chunks], logits for the sampled rows.
Projections and the vocabulary head are library GEMMs (torch -> cuBLAS); everything between them is this repo's kernels
(csrc/group_norm.cu, delta_rule.cu, chunk_attention.cu, moe.cu, post_norm.cu).  There is no CPU path.

Every size, the layer order and every constant come from the checkpoint's config.json (`architecture: "Tonilix"`), the
ranks of the low-rank projections from the tensors' shapes; weights from its *.safetensors, or random from a seed.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Optional, Tuple, Union

import torch

from . import ops

ARCHITECTURE = "Tonilix"
UNIT_EPS = 1e-6            # the design fixes the eps under the root of the unit-vector step
SINUSOID_BASE = 10000.0    # ... and the base of the positional frequencies


@dataclass
class DeltaSpec:
    heads: int
    kv_heads: int
    dim: int                   # per-head query / key size
    vdim: int                  # per-head value size
    taps: int                  # short convolution length
    decay_rank: int = 16       # inner size of the low-rank decay projection
    gate_rank: int = 16        # inner size of the low-rank output-gate projection


@dataclass
class AttnSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    temp_coef: float = 0.0     # query factor 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)
    temp_every: int = 1


@dataclass
class LinearSpec:
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: int = 16


@dataclass
class ParallelSpec:
    left: AttnSpec
    right: LinearSpec
    left_scale: float
    right_scale: float


@dataclass
class DenseSpec:
    ff: int


@dataclass
class ExpertsSpec:
    experts: int
    top: int
    ff: int
    groups: int = 1
    keep: int = 1
    scale: float = 1.0


@dataclass
class LayerSpec:
    mixer: Union[DeltaSpec, ParallelSpec]
    mlp: Union[None, DenseSpec, ExpertsSpec]


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


@dataclass
class TonilixConfig:
    name: str
    vocab: int
    hidden: int
    layer_specs: List[LayerSpec]
    eps: float = 1e-6
    groups: int = 1                        # parts of the RMS norm
    max_position: int = 1 << 20            # positions are computed, not looked up: only the cache bounds a sequence
    family: str = "tonilix"

    @property
    def layers(self) -> int:
        return len(self.layer_specs)

    @property
    def params(self) -> int:
        D = self.hidden
        n = 2 * self.vocab * D + 2 * D
        for L in self.layer_specs:
            m = L.mixer
            n += 3 * D
            if isinstance(m, DeltaSpec):
                C = 2 * m.kv_heads * m.dim + m.heads * m.vdim
                n += D * (C + m.heads + m.decay_rank + m.gate_rank) + C * m.taps + m.decay_rank * m.heads * m.dim \
                    + m.gate_rank * m.heads * m.vdim + m.heads * (1 + m.dim) + m.vdim + m.heads * m.vdim * D
            else:
                a, b = m.left, m.right
                n += (D + 1) * (a.heads * a.dim + a.kv_heads * (a.dim + a.vdim)) + 2 * D * a.heads * a.vdim + D
                n += D * (2 * b.heads * b.dim + 3 * b.heads * b.vdim + b.decay_rank) + (b.decay_rank + 1) * b.heads * b.dim + b.vdim
            if isinstance(L.mlp, DenseSpec):
                n += 3 * D * L.mlp.ff + 2 * D
            elif L.mlp is not None:
                n += L.mlp.experts * (2 * L.mlp.ff * D + D + 1) + 2 * D
        return n

    def kv_bytes_per_token(self, kv_elem_bytes: int = 2, tp: int = 1) -> int:
        return sum((L.mixer.left.dim + L.mixer.left.vdim) * L.mixer.left.kv_heads * kv_elem_bytes
                   for L in self.layer_specs if isinstance(L.mixer, ParallelSpec))

    def state_bytes_per_seq(self, elem_bytes: int = 2) -> int:
        n = 0
        for L in self.layer_specs:
            m = L.mixer
            n += self.hidden * 4                                    # the token-shift row
            if isinstance(m, DeltaSpec):
                n += m.heads * m.dim * m.vdim * 4 + (m.taps - 1) * (2 * m.kv_heads * m.dim + m.heads * m.vdim) * elem_bytes
            else:
                n += m.right.heads * m.right.dim * m.right.vdim * 4
        return n

    def activation_bytes(self, tokens: int, seqs: int, elem_bytes: int = 2) -> int:
        wide = [self.hidden]
        for L in self.layer_specs:
            m = L.mixer
            if isinstance(m, DeltaSpec):
                C = 2 * m.kv_heads * m.dim + m.heads * m.vdim
                wide.append(3 * C + 2 * m.heads * m.dim + 3 * m.heads * m.vdim)
            else:
                a, b = m.left, m.right
                wide.append(2 * a.heads * (a.dim + 2 * a.vdim) + 3 * (2 * b.heads * b.dim + 2 * b.heads * b.vdim))
            if isinstance(L.mlp, DenseSpec):
                wide.append(3 * L.mlp.ff)
        moe = max([0] + [L.mlp.top * (L.mlp.ff * elem_bytes + self.hidden * 4) for L in self.layer_specs
                         if isinstance(L.mlp, ExpertsSpec)])
        return tokens * (self.hidden * 12 + 4 * max(wide) + 2 * moe) + seqs * self.vocab * 8 + (1 << 28)

    def build_model(self, device, **kw):
        return TonilixModel(self, device, **kw)


def config_from_dict(c: dict, name: str = ARCHITECTURE, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> TonilixConfig:
    """config.json -> TonilixConfig.  Keys: vocab, width, norm {eps, groups}, layers [{type: channel_delta | parallel,
    mixer, mlp null | {kind: dense, ff} | {kind: moe, expert {ff}, router {experts, top, scale, groups {count, keep}}}}];
    a channel_delta mixer: {heads, kv_heads, dim, vdim, conv}; a parallel mixer: {left {heads, kv_heads, dim, vdim, scale,
    q_temp {coef, every}}, right {heads, dim, vdim, tau}, left_scale, right_scale}.  `shapes` (tensor name -> shape of the
    checkpoint) gives the inner sizes of the low-rank projections; without it they come from the optional keys
    decay_rank / gate_rank or default to 16."""
    shapes = shapes or {}

    def rank(tensor: str, m: dict, key: str) -> int:
        if tensor in shapes:
            return int(shapes[tensor][0])
        return int(m.get(key, 16))

    specs: List[LayerSpec] = []
    D = int(c["width"])
    for i, L in enumerate(c["layers"]):
        m, kind = L["mixer"], L["type"]
        if kind == "channel_delta":
            heads = int(m["heads"])
            mixer = DeltaSpec(heads, int(m.get("kv_heads", heads)), int(m["dim"]), int(m.get("vdim", m["dim"])),
                              int(m.get("conv", 1)), rank(f"l{i}.mix.a1", m, "decay_rank"), rank(f"l{i}.mix.g1", m, "gate_rank"))
            if mixer.heads % mixer.kv_heads:
                raise ValueError(f"layer {i}: heads {mixer.heads} not a multiple of kv_heads {mixer.kv_heads}")
            if not 1 <= mixer.taps <= 16:
                raise ValueError(f"layer {i}: convolution of {mixer.taps} taps (1 .. 16)")
        elif kind == "parallel":
            a, b = m["left"], m["right"]
            qt = a.get("q_temp") or {}
            heads = int(a["heads"])
            left = AttnSpec(heads, int(a.get("kv_heads", heads)), int(a["dim"]), int(a.get("vdim", a["dim"])),
                            float(a.get("scale", int(a["dim"]) ** -0.5)), float(qt.get("coef", 0.0)), int(qt.get("every", 1)))
            if left.heads % left.kv_heads:
                raise ValueError(f"layer {i}: heads {left.heads} not a multiple of kv_heads {left.kv_heads}")
            if left.temp_coef != 0.0 and left.temp_every < 1:
                raise ValueError(f"layer {i}: q_temp.every must be at least 1")
            right = LinearSpec(int(b["heads"]), int(b["dim"]), int(b.get("vdim", b["dim"])), float(b["tau"]),
                               rank(f"l{i}.mix.right.a1", b, "decay_rank"))
            if right.tau <= 0:
                raise ValueError(f"layer {i}: tau must be positive")
            mixer = ParallelSpec(left, right, float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0)))
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        f = L.get("mlp")
        mlp: Union[None, DenseSpec, ExpertsSpec] = None
        if f:
            fk = f.get("kind")
            if fk == "dense":
                mlp = DenseSpec(int(f["ff"]))
            elif fk == "moe":
                r = f["router"]
                g = r.get("groups") or {}
                mlp = ExpertsSpec(int(r["experts"]), int(r["top"]), int(f["expert"]["ff"]), int(g.get("count", 1)),
                                  int(g.get("keep", g.get("count", 1))), float(r.get("scale", 1.0)))
                if not 1 <= mlp.top <= mlp.experts:
                    raise ValueError(f"layer {i}: router picks {mlp.top} of {mlp.experts} experts")
                if mlp.groups < 1 or mlp.experts % mlp.groups or not 1 <= mlp.keep <= mlp.groups:
                    raise ValueError(f"layer {i}: {mlp.experts} experts in {mlp.groups} groups of which {mlp.keep} are kept")
                if mlp.keep * (mlp.experts // mlp.groups) < mlp.top:
                    raise ValueError(f"layer {i}: {mlp.keep} groups of {mlp.experts // mlp.groups} experts cannot give {mlp.top}")
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {fk!r}")
        specs.append(LayerSpec(mixer, mlp))
    norm = c.get("norm") or {}
    groups = int(norm.get("groups", 1))
    if groups < 1 or D % groups:
        raise ValueError(f"width {D} is not a multiple of {groups} norm groups")
    return TonilixConfig(name=name, vocab=int(c["vocab"]), hidden=D, layer_specs=specs, eps=float(norm.get("eps", 1e-6)),
                         groups=groups)


def safetensors_shapes(path: Path) -> Dict[str, Tuple[int, ...]]:
    """Tensor name -> shape from the headers of a directory's *.safetensors (8-byte little-endian length, then JSON)."""
    out: Dict[str, Tuple[int, ...]] = {}
    for f in sorted(Path(path).glob("*.safetensors")):
        with open(f, "rb") as fh:
            (n,) = struct.unpack("<Q", fh.read(8))
            head = json.loads(fh.read(n))
        for k, v in head.items():
            if k != "__metadata__":
                out[k] = tuple(v["shape"])
    return out


def config_from_dir(path: Path) -> TonilixConfig:
    return config_from_dict(json.loads((Path(path) / "config.json").read_text()), name=Path(path).name,
                            shapes=safetensors_shapes(Path(path)))


def bench_config(hidden: int, layers: int, heads: int, kv_heads: int, head_dim: int, ff: int, experts: int, top: int,
                 vocab: int, taps: int = 4, rank: int = 64, name: str = "tonilix-bench") -> TonilixConfig:
    """A model-sized geometry for benchmarks: parallel and channel_delta layers alternate (parallel first); layer 0 has
    a dense feed-forward of the experts' active width, the rest are routed."""
    specs = []
    for i in range(layers):
        if i % 2 == 0:
            m = ParallelSpec(AttnSpec(heads, kv_heads, head_dim, head_dim, head_dim ** -0.5, 0.25, 512),
                             LinearSpec(max(heads // 2, 1), head_dim, head_dim, 8.0, rank), 1.0, 1.0)
        else:
            m = DeltaSpec(heads, kv_heads, head_dim, head_dim, taps, rank, rank)
        groups = 8 if experts % 8 == 0 and experts // 2 >= top else 1
        specs.append(LayerSpec(m, DenseSpec(ff * top) if i == 0 else ExpertsSpec(experts, top, ff, groups, max(groups // 2, 1), 2.0)))
    return TonilixConfig(name, vocab, hidden, specs, groups=8 if hidden % 8 == 0 else 1)


class TonilixModel:
    """Weights + per-layer caches and states + forward over one scheduled token batch.  One instance per GPU."""

    supports_fp32 = True
    launches_per_layer = 14

    def __init__(self, cfg: TonilixConfig, device: torch.device, num_blocks: int, block_size: int = 16, seed: int = 0,
                 weights_dir: Optional[Path] = None, max_position: Optional[int] = None,
                 kv_dtype: torch.dtype = torch.bfloat16, tp=None, dtype: torch.dtype = torch.bfloat16,
                 max_num_seqs: int = 1):
        if device.type != "cuda":
            raise ValueError("TonilixModel needs a CUDA device (b200attn has no CPU path)")
        if tp is not None and tp.size > 1:
            raise ValueError("Tonilix runs on one GPU per replica: tensor_parallel_size must be 1")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {dtype}: bfloat16 or float32")
        if kv_dtype not in (torch.bfloat16, dtype):
            raise ValueError("Tonilix keeps its K/V pools in the activation type (no fp8 cache)")
        self.cfg, self.dev, self.bs, self.dtype = cfg, device, block_size, dtype
        self.tp, self.tp_size, self.tp_rank = None, 1, 0
        self.vocab_parallel = False
        self.Hq = self.Hkv = 0                      # no paged-decode schedule to plan
        self.max_position = max_position or cfg.max_position
        self.max_num_seqs = max_num_seqs
        self.w: Dict[str, torch.Tensor] = {}
        self.cols: Dict[int, Dict[str, int]] = {}   # layer -> first column of every part of its fused projection
        if weights_dir is not None and any(Path(weights_dir).glob("*.safetensors")):
            self._load(Path(weights_dir))
        else:
            self._random_init(seed)
        self._fuse()
        self.freq = ops.sinusoid_frequencies(cfg.hidden, SINUSOID_BASE, device)
        self.num_blocks = 0
        self.k_cache: Dict[int, torch.Tensor] = {}
        self.v_cache: Dict[int, torch.Tensor] = {}
        self.state: Dict[int, torch.Tensor] = {}
        self.conv_state: Dict[int, torch.Tensor] = {}
        self.shift_state: Dict[int, torch.Tensor] = {}
        self.alloc_cache(num_blocks)
        self.alloc_state(max_num_seqs)
        self._arange = torch.arange(max_num_seqs + 1, dtype=torch.int32, device=device)
        # the two halves of a parallel mixer are independent between the fused projection and the output projection: the
        # recurrent half (few CTAs, a long dependent chain per sequence) runs on a second stream under the attention
        self.overlap = os.environ.get("B2_PARALLEL_MIXER_STREAMS", "1") != "0"
        self._side = torch.cuda.Stream(device)
        # heads of 128 in bf16 are what the Llama path's attention kernels are built for (tcgen05 prompt chunks, TMA paged
        # decode): a parallel mixer with such heads runs on them when the full library is loaded
        from . import _lib
        self._llama_attention = dtype == torch.bfloat16 and block_size in (8, 16, 32) and _lib.is_full() \
            and os.environ.get("B2_TONILIX_LLAMA_ATTENTION", "1") != "0"
        self.capture: Optional[list] = None         # tests: set to a list to collect the residual after every layer

    # ------------------------------------------------------------------ weights
    def _tensor_names(self) -> Dict[str, Tuple[int, ...]]:
        """Name -> shape of every tensor of a checkpoint of this configuration."""
        c, D = self.cfg, self.cfg.hidden
        out = {"embed": (c.vocab, D), "embed.norm": (D,), "final.norm": (D,), "head": (c.vocab, D)}
        for i, L in enumerate(c.layer_specs):
            p, m, f = f"l{i}", L.mixer, L.mlp
            out.update({p + ".norm1": (D,), p + ".ls1": (D,), p + ".shift": (D,)})
            if isinstance(m, DeltaSpec):
                q, Gk, Hv = p + ".mix", m.kv_heads * m.dim, m.heads * m.vdim
                out.update({q + ".q": (Gk, D), q + ".k": (Gk, D), q + ".v": (Hv, D), q + ".q.conv": (Gk, m.taps),
                            q + ".k.conv": (Gk, m.taps), q + ".v.conv": (Hv, m.taps), q + ".b": (m.heads, D),
                            q + ".A_log": (m.heads,), q + ".norm": (m.vdim,), q + ".a1": (m.decay_rank, D),
                            q + ".a2": (m.heads * m.dim, m.decay_rank), q + ".dt_bias": (m.heads * m.dim,),
                            q + ".g1": (m.gate_rank, D), q + ".g2": (Hv, m.gate_rank), q + ".o": (D, Hv)})
            else:
                a, b = m.left, m.right
                q = p + ".mix.left"
                for n, rows in (("q", a.heads * a.dim), ("k", a.kv_heads * a.dim), ("v", a.kv_heads * a.vdim)):
                    out[f"{q}.{n}"] = (rows, D)
                    out[f"{q}.{n}.b"] = (rows,)
                out.update({q + ".g": (a.heads * a.vdim, D), q + ".o": (D, a.heads * a.vdim), q + ".o.b": (D,)})
                q = p + ".mix.right"
                out.update({q + ".q": (b.heads * b.dim, D), q + ".k": (b.heads * b.dim, D), q + ".v": (b.heads * b.vdim, D),
                            q + ".g": (b.heads * b.vdim, D), q + ".o": (D, b.heads * b.vdim), q + ".norm": (b.vdim,),
                            q + ".a1": (b.decay_rank, D), q + ".a2": (b.heads * b.dim, b.decay_rank),
                            q + ".a2.b": (b.heads * b.dim,)})
            if f is not None:
                out.update({p + ".norm2": (D,), p + ".ls2": (D,)})
            if isinstance(f, DenseSpec):
                out.update({p + ".mlp.gate": (f.ff, D), p + ".mlp.up": (f.ff, D), p + ".mlp.down": (D, f.ff)})
            elif f is not None:
                for e in range(f.experts):
                    out.update({f"{p}.mlp.e{e}.up": (f.ff, D), f"{p}.mlp.e{e}.down": (D, f.ff)})
                out.update({p + ".mlp.router": (f.experts, D), p + ".mlp.correction": (f.experts,)})
        return out

    def _random_init(self, seed: int) -> None:
        g = torch.Generator(device=self.dev).manual_seed(seed)
        raw = {}
        for name, shape in self._tensor_names().items():
            leaf = name.rsplit(".", 1)[-1]
            t = torch.randn(*shape, generator=g, device=self.dev, dtype=torch.float32)
            if leaf == "A_log":
                t = 0.5 * t - 1.0
            elif name.endswith(".a2.b"):
                t = 0.5 * t + 2.0
            elif leaf in ("dt_bias", "correction"):
                t = 0.3 * t
            elif leaf == "b" and len(shape) == 1:
                t = 0.1 * t
            elif leaf == "shift":
                t = 0.5 * torch.sigmoid(t)
            elif leaf == "conv":
                t = t * shape[1] ** -0.5
            elif len(shape) == 1:
                t = 1.0 + 0.1 * t
            elif name != "embed":
                t = t * shape[-1] ** -0.5
            raw[name] = t.to(torch.bfloat16)
        self._ingest(raw)

    def _load(self, path: Path) -> None:
        from safetensors import safe_open
        raw: Dict[str, torch.Tensor] = {}
        for f in sorted(path.glob("*.safetensors")):
            with safe_open(str(f), framework="pt", device="cpu") as sf:
                for k in sf.keys():
                    raw[k] = sf.get_tensor(k)
        want = self._tensor_names()
        missing = [k for k in want if k not in raw]
        if missing:
            raise ValueError(f"checkpoint lacks {len(missing)} tensors, e.g. {missing[:3]}")
        for k, shape in want.items():
            if tuple(raw[k].shape) != tuple(shape):
                raise ValueError(f"{k}: shape {tuple(raw[k].shape)} in the checkpoint, {tuple(shape)} by config.json")
        self._ingest({k: raw[k].to(self.dev) for k in want})

    def _ingest(self, raw: Dict[str, torch.Tensor]) -> None:
        """Matrices and projection biases in the activation type, parameter vectors and convolution taps in fp32."""
        for k, t in raw.items():
            proj_bias = k.endswith((".q.b", ".k.b", ".v.b"))          # added inside the fused projection
            small = (t.dim() == 1 and not proj_bias) or k.endswith(".conv")
            self.w[k] = t.to(torch.float32 if small else self.dtype).contiguous()

    def _stack(self, li: int, parts: List[Tuple[str, List[torch.Tensor]]], D: int) -> torch.Tensor:
        """Rows of several matrices as one projection matrix; every named part starts on a multiple of eight rows (zero
        rows between), so that the columns it produces stay 16-byte aligned.  Records the parts' first columns."""
        rows, cols, at = [], {}, 0
        for name, mats in parts:
            cols[name] = at
            n = sum(m.shape[0] for m in mats)
            rows += mats
            pad = _pad8(n) - n
            if pad:
                rows.append(torch.zeros(pad, D, dtype=self.dtype, device=self.dev))
            at += n + pad
        self.cols[li] = cols
        return torch.cat(rows).contiguous()

    def _fuse(self) -> None:
        """Per layer: ONE projection matrix for everything that reads the mixer's input, the second matrices of the low-rank
        projections padded to the aligned inner size, the two output projections of a parallel mixer side by side, gate
        and up of a dense feed-forward stacked, expert matrices stacked."""
        w, c, D = self.w, self.cfg, self.cfg.hidden
        pop = w.pop

        def low_rank_second(name: str, r: int) -> torch.Tensor:
            m = pop(name)
            out = torch.zeros(m.shape[0], _pad8(r), dtype=self.dtype, device=self.dev)
            out[:, :r] = m
            return out

        for i, L in enumerate(c.layer_specs):
            p, m, f = f"l{i}", L.mixer, L.mlp
            if isinstance(m, DeltaSpec):
                q = p + ".mix"
                w[p + ".wproj"] = self._stack(i, [("qkv", [pop(q + ".q"), pop(q + ".k"), pop(q + ".v")]), ("a1", [pop(q + ".a1")]),
                                                  ("g1", [pop(q + ".g1")]), ("b", [pop(q + ".b")])], D)
                w[p + ".conv"] = torch.cat([pop(q + ".q.conv"), pop(q + ".k.conv"), pop(q + ".v.conv")]).contiguous()
                w[q + ".a2"] = low_rank_second(q + ".a2", m.decay_rank)
                w[q + ".g2"] = low_rank_second(q + ".g2", m.gate_rank)
            else:
                a, b = m.left, m.right
                ql, qr = p + ".mix.left", p + ".mix.right"
                names = [ql + ".q", ql + ".k", ql + ".v"]
                bias = torch.cat([pop(n + ".b") for n in names])
                w[p + ".wproj"] = self._stack(i, [("left", [pop(n) for n in names]), ("lgate", [pop(ql + ".g")]),
                                                  ("right", [pop(qr + ".q"), pop(qr + ".k"), pop(qr + ".v")]),
                                                  ("rgate", [pop(qr + ".g")]), ("a1", [pop(qr + ".a1")])], D)
                full = torch.zeros(w[p + ".wproj"].shape[0], dtype=self.dtype, device=self.dev)
                full[:bias.shape[0]] = bias
                w[p + ".bproj"] = full
                w[qr + ".a2"] = low_rank_second(qr + ".a2", b.decay_rank)
                w[p + ".wo"] = torch.cat([pop(ql + ".o"), pop(qr + ".o")], dim=1).contiguous()
                w[p + ".bo"] = (pop(ql + ".o.b") * m.left_scale).contiguous()           # fp32: joins the residual sum
            if isinstance(f, DenseSpec):
                w[p + ".mlp.gate_up"] = torch.cat([pop(p + ".mlp.gate"), pop(p + ".mlp.up")]).contiguous()
            elif f is not None:
                w[p + ".mlp.up"] = torch.stack([pop(f"{p}.mlp.e{e}.up") for e in range(f.experts)]).contiguous()
                w[p + ".mlp.down"] = torch.stack([pop(f"{p}.mlp.e{e}.down") for e in range(f.experts)]).contiguous()

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.w.values())

    # ------------------------------------------------------------------ caches and state
    def alloc_cache(self, num_blocks: int) -> None:
        """K/V pools of every parallel layer's attention: [num_blocks, G, bs, dk] and [num_blocks, G, bs, dv]."""
        self.num_blocks = int(num_blocks)
        self.k_cache.clear(), self.v_cache.clear()
        for i, L in enumerate(self.cfg.layer_specs):
            if isinstance(L.mixer, ParallelSpec):
                a = L.mixer.left
                self.k_cache[i] = torch.zeros(num_blocks, a.kv_heads, self.bs, a.dim, dtype=self.dtype, device=self.dev)
                self.v_cache[i] = torch.zeros(num_blocks, a.kv_heads, self.bs, a.vdim, dtype=self.dtype, device=self.dev)

    def alloc_state(self, max_num_seqs: int) -> None:
        """One slot per live sequence and layer: the token-shift row (fp32), the matrix state of the layer's recurrence
        (fp32) and the convolution tail (activation type).  Slots are never cleared: a sequence that starts at position 0
        ignores their contents."""
        self.max_num_seqs = int(max_num_seqs)
        self.state.clear(), self.conv_state.clear(), self.shift_state.clear()
        for i, L in enumerate(self.cfg.layer_specs):
            m = L.mixer
            self.shift_state[i] = torch.zeros(max_num_seqs, self.cfg.hidden, dtype=torch.float32, device=self.dev)
            if isinstance(m, DeltaSpec):
                C = 2 * m.kv_heads * m.dim + m.heads * m.vdim
                self.state[i] = torch.zeros(max_num_seqs, m.heads, m.dim, m.vdim, dtype=torch.float32, device=self.dev)
                if m.taps > 1:
                    self.conv_state[i] = torch.zeros(max_num_seqs, m.taps - 1, C, dtype=self.dtype, device=self.dev)
            else:
                b = m.right
                self.state[i] = torch.zeros(max_num_seqs, b.heads, b.dim, b.vdim, dtype=torch.float32, device=self.dev)

    def prepare_decode(self, max_batch: int, max_nb: int) -> None:
        """Static index tensors of the decode-only batch (one row per sequence)."""
        if self._arange.shape[0] < max_batch + 1:
            self._arange = torch.arange(max_batch + 1, dtype=torch.int32, device=self.dev)

    def decode_schedule(self, seq_lens_host) -> int:
        return 0

    # ------------------------------------------------------------------ forward
    def _low_rank(self, first: torch.Tensor, second: torch.Tensor, fp32_out: bool) -> torch.Tensor:
        """second @ first-stage outputs; what enters a recurrence comes out of the product in fp32."""
        if fp32_out and first.dtype == torch.bfloat16:
            return torch.mm(first, second.t(), out_dtype=torch.float32)
        return torch.mm(first, second.t())

    def _delta_mixer(self, li: int, h: torch.Tensor, batch: ops.SeqBatch) -> torch.Tensor:
        m, w, p, cols = self.cfg.layer_specs[li].mixer, self.w, f"l{li}", self.cols[li]
        H, G, dk, dv = m.heads, m.kv_heads, m.dim, m.vdim
        proj = torch.nn.functional.linear(h, w[p + ".wproj"])
        a = self._low_rank(proj[:, cols["a1"]:cols["a1"] + _pad8(m.decay_rank)], w[p + ".mix.a2"], True)       # fp32 [T, H*dk]
        gate = self._low_rank(proj[:, cols["g1"]:cols["g1"] + _pad8(m.gate_rank)], w[p + ".mix.g2"], False)
        qkv, beta, decay = ops.recur_prep(proj, H, G, dk, dv, batch, taps=m.taps, conv_w=w[p + ".conv"],
                                          conv_state=self.conv_state.get(li), conv_silu=True, unit=True, unit_eps=UNIT_EPS,
                                          q_scale=dk ** -0.5, off_beta=cols["b"], decay_mode=ops.DECAY_CHANNEL_SOFTPLUS, a=a,
                                          A_log=w[p + ".mix.A_log"], decay_bias=w[p + ".mix.dt_bias"])
        o = ops.channel_scan(qkv, beta, decay, H, G, dk, dv, batch, self.state[li], delta=True)
        out = ops.gated_head_norm(o, gate, w[p + ".mix.norm"], self.cfg.eps, ops.GATE_SIGMOID)
        return torch.nn.functional.linear(out, w[p + ".mix.o"])

    def _parallel_mixer(self, li: int, h: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                        batch: ops.SeqBatch, n_decode: int = 0, dec_bt=None, dec_sl=None, prefill=None) -> torch.Tensor:
        m, w, p, cols = self.cfg.layer_specs[li].mixer, self.w, f"l{li}", self.cols[li]
        a, b = m.left, m.right
        T = h.shape[0]
        proj = torch.nn.functional.linear(h, w[p + ".wproj"], w[p + ".bproj"])
        nl, nr = a.heads * a.vdim, b.heads * b.vdim
        cat = torch.empty(T, nl + nr, dtype=h.dtype, device=h.device)       # [left heads, gated | right heads, normed and gated]

        def right():                                 # gated linear attention over the state slots
            z = self._low_rank(proj[:, cols["a1"]:cols["a1"] + _pad8(b.decay_rank)], w[p + ".mix.right.a2"], True)
            qkv, _, decay = ops.recur_prep(proj[:, cols["right"]:], b.heads, b.heads, b.dim, b.vdim, batch, q_scale=b.dim ** -0.5,
                                           decay_mode=ops.DECAY_CHANNEL_SIGMOID_POW, a=z, decay_bias=w[p + ".mix.right.a2.b"],
                                           tau=b.tau)
            s = ops.channel_scan(qkv, None, decay, b.heads, b.heads, b.dim, b.vdim, batch, self.state[li], delta=False)
            ops.gated_head_norm(s, proj[:, cols["rgate"]:cols["rgate"] + nr], w[p + ".mix.right.norm"], self.cfg.eps,
                                ops.GATE_SILU, m.right_scale, out=cat[:, nl:])

        main = torch.cuda.current_stream(self.dev)
        if self.overlap:
            self._side.wait_stream(main)             # proj and cat exist
            with torch.cuda.stream(self._side):
                right()
        # softmax attention over the paged pools
        wl = a.heads * a.dim + a.kv_heads * (a.dim + a.vdim)
        q = ops.qk_prep_cache(proj[:, :wl], a.heads, a.kv_heads, a.dim, a.vdim, slots, self.k_cache[li], self.v_cache[li],
                              positions, a.temp_coef, a.temp_every)
        if self._llama_attention and a.dim == 128 and a.vdim == 128:
            o = torch.empty(T, a.heads, 128, dtype=h.dtype, device=h.device)
            if n_decode:
                ops.paged_decode(q[:n_decode], self.k_cache[li], self.v_cache[li], dec_bt, dec_sl, scale=a.scale, out=o[:n_decode])
            if prefill is not None and prefill.total_tokens:
                ops.prefill_attention(q[n_decode:], self.k_cache[li], self.v_cache[li], prefill.block_tables, prefill.cu_q,
                                      prefill.ctx_start, total_tokens=prefill.total_tokens, scale=a.scale, out=o[n_decode:])
        else:
            o = ops.chunk_attention(q, self.k_cache[li], self.v_cache[li], batch, a.scale)
        ops.gate_mul(o.view(T, nl), proj[:, cols["lgate"]:cols["lgate"] + nl], ops.GATE_SIGMOID, m.left_scale, out=cat[:, :nl])
        if self.overlap:
            main.wait_stream(self._side)
        else:
            right()
        return torch.nn.functional.linear(cat, w[p + ".wo"])                # + left_scale * o.b, added with the residual

    def _mlp(self, li: int, h: torch.Tensor) -> torch.Tensor:
        f, w, p = self.cfg.layer_specs[li].mlp, self.w, f"l{li}.mlp"
        if isinstance(f, DenseSpec):
            gu = torch.nn.functional.linear(h, w[p + ".gate_up"])
            return torch.nn.functional.linear(ops.glu_and_mul(gu, ops.GLU_GELU_TANH), w[p + ".down"])
        ids, wts = ops.moe_route(h, w[p + ".router"], w[p + ".correction"], f.top, scoring=ops.ROUTE_SIGMOID_GROUPED,
                                 n_groups=f.groups, keep_groups=f.keep, weight_scale=f.scale)
        return ops.moe_experts(h, ids, wts, None, w[p + ".up"], w[p + ".down"], glu=ops.FF_RELU_SQ)

    def forward(self, tokens: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, n_decode: int,
                dec_block_tables: Optional[torch.Tensor], dec_seq_lens: Optional[torch.Tensor], prefill,
                sample_rows: Optional[torch.Tensor], num_splits: int = 0,
                dec_state_slots: Optional[torch.Tensor] = None) -> torch.Tensor:
        """tokens int64 [T] (rows [0, n_decode) = one new token per running sequence, the rest = prompt chunks),
        positions int32 [T], slots int64 [T] (cache slot of every row).  Returns logits [len(sample_rows) or T, vocab]
        in the model's dtype."""
        c, w = self.cfg, self.w
        if n_decode and self._arange.shape[0] < n_decode + 1:
            self._arange = torch.arange(n_decode + 1, dtype=torch.int32, device=self.dev)
        if n_decode and dec_state_slots is None:
            raise ValueError("decode rows need their state slots")
        if prefill is not None and prefill.total_tokens and prefill.state_slots is None:
            raise ValueError("prompt chunks need their state slots")
        batch = ops.step_batch(self._arange, n_decode, dec_block_tables, dec_seq_lens, dec_state_slots, prefill)
        x = ops.embed_sinusoid_norm(w["embed"], tokens, positions, self.freq, w["embed.norm"], c.groups, c.eps)
        spare = torch.empty_like(x)                  # a sublayer output lands here when the next read-out is shifted
        n = len(c.layer_specs)
        h = ops.group_norm_step(x, norm_w=w["l0.norm1"], groups=c.groups, eps=c.eps, h_dtype=self.dtype, shift_mu=w["l0.shift"],
                                shift_state=self.shift_state[0], batch=batch)
        for li in range(n):
            p, L = f"l{li}", c.layer_specs[li]
            if isinstance(L.mixer, DeltaSpec):
                y, ybias = self._delta_mixer(li, h, batch), None
            else:
                y = self._parallel_mixer(li, h, positions, slots, batch, n_decode, dec_block_tables, dec_seq_lens, prefill)
                ybias = w[p + ".bo"]
            scale = w[p + ".ls1"]
            if L.mlp is not None:
                h = ops.group_norm_step(x, y, scale, ybias, w[p + ".norm2"], c.groups, c.eps, h_dtype=self.dtype)
                y, ybias, scale = self._mlp(li, h), None, w[p + ".ls2"]
            if li + 1 < n:
                q = f"l{li + 1}"
                h = ops.group_norm_step(x, y, scale, ybias, w[q + ".norm1"], c.groups, c.eps, h_dtype=self.dtype,
                                        shift_mu=w[q + ".shift"], shift_state=self.shift_state[li + 1], batch=batch, x_out=spare)
                x, spare = spare, x
            else:
                ops.group_norm_step(x, y, scale, ybias)
            if self.capture is not None:
                self.capture.append(x.clone())
        if sample_rows is not None:
            x = x.index_select(0, sample_rows).contiguous()
        h = ops.group_norm_step(x, norm_w=w["final.norm"], groups=c.groups, eps=c.eps, h_dtype=self.dtype)
        return torch.nn.functional.linear(h, w["head"])
