"""Sanarax decoder on the b200attn ops: layers with an RMS norm (weight stored around zero, applied as 1 + w) before AND
after every sublayer around one fp32 residual, and one of three sequence mixers per layer:

  lightning          linear attention with one fixed decay per head, S <- decay_h S + k v^T, o = S^T q over SiLU-activated
                     q, k, v; the concatenated heads are RMS-normed as one row, gated by a sigmoid per channel.  The matrix
                     state lives in fp32 state slots, one per live sequence and layer.
  attention          grouped-query softmax attention whose values are the keys as projected (before their rotation), with
                     biased projections, a partial rotation in the (i, i + dims/2) layout, a sliding window that keeps the
                     sequence's first tokens, a learned sink per head in the denominator and a sigmoid gate per head.
  latent_attention   causal softmax attention over one low-rank latent per token that all heads share plus one shared
                     rotated key part (interleaved pairs); the queries come through a normalised latent of their own.

The feed-forward is dense with a squared ReLU, or absent.  A layer may use another layer's tensors (`weights_of`) with a
cache or state of its own.  The embedding and the logits carry fixed factors.

The model plugs into the same engine as the other families (b200attn.engine.LLMEngine): paged pools addressed through the
scheduler's block tables and slot mapping, state slots per live sequence, one forward over [decode rows | prompt chunks],
logits for the sampled rows.  Projections and the vocabulary head are library GEMMs (torch -> cuBLAS); everything between
them is this repo's kernels (csrc/post_norm.cu, chunk_attention.cu, latent_attention.cu, delta_rule.cu).  There is no CPU
path.

Every size, the layer order and every constant come from the checkpoint's config.json (`architecture: "Sanarax"`);
weights from its *.safetensors, or random from a seed.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Optional, Tuple, Union

import torch

from . import ops

ARCHITECTURE = "Sanarax"
# A step with at least this many prompt rows rebuilds keys and values per head for them in its latent layers (bf16):
# (dim + rot_dim + vdim) multiplications per (query, key, head) instead of (2 kv_rank + rot_dim) in the latent space, for
# two more GEMMs per layer over the rows the portions can see.  Decode rows and short portions stay in the latent space.
PROMPT_PER_HEAD_MIN_ROWS = 256
PROMPT_PER_HEAD_MAX_CONTEXT = 4      # ... unless the visible rows outnumber the prompt rows by more than this factor


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


@dataclass(frozen=True)
class LightningSpec:
    heads: int
    dim: int                   # per-head query / key size
    vdim: int                  # per-head value size
    decay: Tuple[float, ...]   # one fixed factor per head


@dataclass(frozen=True)
class WindowSpec:
    heads: int
    kv_heads: int
    dim: int                   # per-head query / key size; the values are the keys, so also the value size
    scale: float
    window: int = 0            # a query sees its own position and the window - 1 before it (0: plain causal) ...
    keep_first: int = 0        # ... and the first keep_first positions of the sequence
    rot_dims: int = 0          # how many leading entries of a head turn (the rest pass)
    rot_base: float = 10000.0


@dataclass(frozen=True)
class LatentSpec:
    heads: int
    dim: int                   # per-head unrotated query / key size
    rot_dim: int               # per-head rotated query size = size of the shared rotated key part
    vdim: int
    kv_rank: int               # key / value latent size
    q_rank: int                # query latent size
    scale: float
    rot_dims: int = 0
    rot_base: float = 10000.0

    @property
    def row(self) -> int:
        return self.kv_rank + self.rot_dim


@dataclass(frozen=True)
class DenseSpec:
    ff: int


MixerSpec = Union[LightningSpec, WindowSpec, LatentSpec]


@dataclass
class LayerSpec:
    mixer: MixerSpec
    mlp: Optional[DenseSpec]
    weights: int               # the layer whose tensors this layer uses (itself unless config.json says weights_of)


@dataclass
class SanaraxConfig:
    name: str
    vocab: int
    hidden: int
    layer_specs: List[LayerSpec]
    eps: float = 1e-6
    embed_scale: float = 1.0
    logit_scale: float = 1.0
    max_position: int = 1 << 20            # the rotary tables are built for the engine's max_model_len
    family: str = "sanarax"

    @property
    def layers(self) -> int:
        return len(self.layer_specs)

    @property
    def params(self) -> int:
        D = self.hidden
        n = 2 * self.vocab * D + D
        for i, L in enumerate(self.layer_specs):
            if L.weights != i:
                continue
            m = L.mixer
            n += 2 * D
            if isinstance(m, LightningSpec):
                n += D * m.heads * (2 * m.dim + 2 * m.vdim) + m.heads * m.vdim * (D + 1)
            elif isinstance(m, WindowSpec):
                n += (D + 1) * (m.heads + m.kv_heads) * m.dim + m.heads * (D + 1) + m.heads * m.dim * D
            else:
                n += D * (m.q_rank + m.row + m.heads) + m.q_rank * (1 + m.heads * (m.dim + m.rot_dim)) + m.kv_rank \
                    + m.kv_rank * m.heads * (m.dim + m.vdim) + m.heads * m.vdim * D
            if L.mlp is not None:
                n += 2 * D * L.mlp.ff + 2 * D
        return n

    def kv_bytes_per_token(self, kv_elem_bytes: int = 2, tp: int = 1) -> int:
        n = 0
        for L in self.layer_specs:                   # every layer RUN has a pool of its own, shared tensors or not
            m = L.mixer
            if isinstance(m, WindowSpec):
                n += 2 * m.kv_heads * m.dim * kv_elem_bytes
            elif isinstance(m, LatentSpec):
                n += m.row * kv_elem_bytes
        return n

    def state_bytes_per_seq(self, elem_bytes: int = 2) -> int:
        return sum(L.mixer.heads * L.mixer.dim * L.mixer.vdim * 4 for L in self.layer_specs if isinstance(L.mixer, LightningSpec))

    def activation_bytes(self, tokens: int, seqs: int, elem_bytes: int = 2) -> int:
        wide = [self.hidden]
        for L in self.layer_specs:
            m = L.mixer
            if isinstance(m, LightningSpec):
                wide.append(m.heads * (2 * m.dim + 2 * m.vdim) * 3)          # projection rows + their fp32 copy for the scan
            elif isinstance(m, WindowSpec):
                wide.append((2 * m.heads + m.kv_heads) * m.dim + m.heads)
            else:
                wide.append(m.q_rank + m.row + m.heads * (m.dim + m.rot_dim + 1 + 2 * m.row + m.vdim))
            if L.mlp is not None:
                wide.append(2 * L.mlp.ff)
        return tokens * (self.hidden * 8 + 2 * max(wide) * elem_bytes) + seqs * self.vocab * 8 + (1 << 28)

    def build_model(self, device, **kw):
        return SanaraxModel(self, device, **kw)


def _rot(m: dict, default_dims: int) -> Tuple[int, float]:
    rot = m.get("rot") or {}
    return int(rot.get("dims", default_dims)), float(rot.get("base", 10000.0))


def config_from_dict(c: dict, name: str = ARCHITECTURE, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> SanaraxConfig:
    """config.json -> SanaraxConfig.  Keys: vocab, width, norm.eps, embedding.scale, logit_scale, layers [{type, mixer,
    mlp null | {kind: dense, ff}, weights_of}] with the mixers
      lightning         {heads, dim, vdim, decay [heads]}
      attention         {heads, kv_heads, dim, vdim (= dim), scale, mask {size, keep_first}, rot {base, dims}}
      latent_attention  {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot {base, dims}}.
    `shapes` (tensor name -> shape from the checkpoint's header) supplies q_rank when config.json leaves it out."""
    specs: List[LayerSpec] = []
    raw = c["layers"]
    for i, L in enumerate(raw):
        src = i if L.get("weights_of") is None else int(L["weights_of"])
        if src != i and 0 <= src < len(raw):         # what such an entry leaves out is the owner's
            L = {**raw[src], **L}
        kind, m = L["type"], L["mixer"]
        if kind == "lightning":
            mixer: MixerSpec = LightningSpec(int(m["heads"]), int(m["dim"]), int(m["vdim"]), tuple(float(x) for x in m["decay"]))
            if len(mixer.decay) != mixer.heads:
                raise ValueError(f"layer {i}: {len(mixer.decay)} decay factors for {mixer.heads} heads")
        elif kind == "attention":
            mask = m.get("mask") or {}
            dims, base = _rot(m, 0)
            mixer = WindowSpec(int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), float(m["scale"]),
                               int(mask.get("size") or 0), int(mask.get("keep_first") or 0), dims, base)
            if int(m.get("vdim", mixer.dim)) != mixer.dim:
                raise ValueError(f"layer {i}: the values are the keys, vdim {m['vdim']} must equal dim {mixer.dim}")
            if mixer.kv_heads < 1 or mixer.heads % mixer.kv_heads:
                raise ValueError(f"layer {i}: {mixer.heads} query heads over {mixer.kv_heads} key/value heads")
            if dims % 2 or not 0 <= dims <= mixer.dim:
                raise ValueError(f"layer {i}: rot.dims {dims} must be even and at most dim {mixer.dim}")
        elif kind == "latent_attention":
            rot_dim = int(m["rot_dim"])
            dims, base = _rot(m, rot_dim)
            q_rank = m.get("q_rank")
            if q_rank is None:
                if not shapes or f"l{src}.mix.dq" not in shapes:
                    raise ValueError(f"layer {i}: q_rank is neither in config.json nor readable from the checkpoint")
                q_rank = shapes[f"l{src}.mix.dq"][0]
            mixer = LatentSpec(int(m["heads"]), int(m["dim"]), rot_dim, int(m["vdim"]), int(m["kv_rank"]), int(q_rank),
                               float(m["scale"]), dims, base)
            if dims % 2 or not 0 <= dims <= rot_dim:
                raise ValueError(f"layer {i}: rot.dims {dims} must be even and at most rot_dim {rot_dim}")
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        f = L.get("mlp")
        mlp = None
        if f:
            if f.get("kind") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")
            mlp = DenseSpec(int(f["ff"]))
        specs.append(LayerSpec(mixer, mlp, src))
    for i, L in enumerate(specs):
        if L.weights != i:
            j = L.weights
            if not 0 <= j < len(specs) or specs[j].weights != j:
                raise ValueError(f"layer {i}: weights_of {j} must name a layer with tensors of its own")
            if (specs[j].mixer, specs[j].mlp) != (L.mixer, L.mlp):
                raise ValueError(f"layer {i}: its mixer and feed-forward differ from layer {j}, whose tensors it uses")
    return SanaraxConfig(name=name, vocab=int(c["vocab"]), hidden=int(c["width"]), layer_specs=specs,
                         eps=float((c.get("norm") or {}).get("eps", 1e-6)),
                         embed_scale=float((c.get("embedding") or {}).get("scale", 1.0)),
                         logit_scale=float(c.get("logit_scale", 1.0)))


def config_from_dir(path: Path) -> SanaraxConfig:
    from .tonilix import safetensors_shapes
    path = Path(path)
    return config_from_dict(json.loads((path / "config.json").read_text()), name=path.name, shapes=safetensors_shapes(path))


def bench_config(hidden: int, layers: int, heads: int, kv_heads: int, head_dim: int, ff: int, vocab: int, kv_rank: int = 512,
                 q_rank: int = 1536, rot_dim: int = 64, window: int = 1024, keep_first: int = 4,
                 name: str = "sanarax-bench") -> SanaraxConfig:
    """A model-sized geometry for benchmarks: attention, latent_attention and lightning layers in turn; the lightning
    layers carry no feed-forward, the second half of the stack uses the first half's tensors."""
    specs = []
    for i in range(layers):
        kind = i % 3
        if kind == 0:
            m: MixerSpec = WindowSpec(heads, kv_heads, head_dim, head_dim ** -0.5, window, keep_first, head_dim // 2, 1e6)
        elif kind == 1:
            m = LatentSpec(heads, head_dim, rot_dim, head_dim, kv_rank, q_rank, (head_dim + rot_dim) ** -0.5, rot_dim, 1e4)
        else:
            m = LightningSpec(heads, head_dim, head_dim, tuple(1.0 - 2.0 ** (-5.0 - 3.0 * h / max(heads - 1, 1)) for h in range(heads)))
        half = layers - layers % 6
        src = i - half // 2 if half and half // 2 <= i < half else i
        specs.append(LayerSpec(m, None if kind == 2 else DenseSpec(ff), src))
    return SanaraxConfig(name, vocab, hidden, specs, embed_scale=hidden ** 0.5, logit_scale=hidden ** -0.5)


class SanaraxModel:
    """Weights + per-layer pools and states + forward over one scheduled token batch.  One instance per GPU."""

    supports_fp32 = True
    launches_per_layer = 9

    def __init__(self, cfg: SanaraxConfig, device: torch.device, num_blocks: int, block_size: int = 16, seed: int = 0,
                 weights_dir: Optional[Path] = None, max_position: Optional[int] = None,
                 kv_dtype: torch.dtype = torch.bfloat16, tp=None, dtype: torch.dtype = torch.bfloat16,
                 max_num_seqs: int = 1):
        if device.type != "cuda":
            raise ValueError("SanaraxModel needs a CUDA device (b200attn has no CPU path)")
        if tp is not None and tp.size > 1:
            raise ValueError("Sanarax runs on one GPU per replica: tensor_parallel_size must be 1")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {dtype}: bfloat16 or float32")
        if kv_dtype not in (torch.bfloat16, dtype):
            raise ValueError("Sanarax keeps its pools in the activation type (no fp8 cache)")
        self.cfg, self.dev, self.bs, self.dtype = cfg, device, block_size, dtype
        self.tp, self.tp_size, self.tp_rank = None, 1, 0
        self.vocab_parallel = False
        self.Hq = self.Hkv = 0                      # no paged-decode schedule to plan
        self.max_position = max_position or min(cfg.max_position, 1 << 17)
        self.max_num_seqs = max_num_seqs
        self.w: Dict[str, torch.Tensor] = {}
        self.cols: Dict[int, Dict[str, int]] = {}   # weight layer -> first column of every part of its fused projection
        if weights_dir is not None and any(Path(weights_dir).glob("*.safetensors")):
            self._load(Path(weights_dir))
        else:
            self._random_init(seed)
        self._fuse()
        # one rotary table per distinct (dims, base); both pair layouts read the same table
        self.rot: Dict[tuple, torch.Tensor] = {}
        for L in cfg.layer_specs:
            m = L.mixer
            if not isinstance(m, LightningSpec) and m.rot_dims and (m.rot_dims, m.rot_base) not in self.rot:
                self.rot[(m.rot_dims, m.rot_base)] = ops.rotary_table(self.max_position, m.rot_dims, m.rot_base, None, device)
        self.num_blocks = 0
        self.k_cache: Dict[int, torch.Tensor] = {}
        self.v_cache: Dict[int, torch.Tensor] = {}
        self.latent_cache: Dict[int, torch.Tensor] = {}
        self.state: Dict[int, torch.Tensor] = {}
        self.alloc_cache(num_blocks)
        self.alloc_state(max_num_seqs)
        self._arange = torch.arange(max_num_seqs + 1, dtype=torch.int32, device=device)
        self.capture: Optional[list] = None         # tests: set to a list to collect the residual after every layer

    # ------------------------------------------------------------------ weights
    def _tensor_names(self) -> Dict[str, Tuple[int, ...]]:
        """Name -> shape of every tensor of a checkpoint of this configuration (layers that use another layer's have none)."""
        c, D = self.cfg, self.cfg.hidden
        out = {"embed": (c.vocab, D), "final.norm": (D,), "head": (c.vocab, D)}
        for i, L in enumerate(c.layer_specs):
            if L.weights != i:
                continue
            p, m, f = f"l{i}", L.mixer, L.mlp
            q = p + ".mix"
            out.update({p + ".norm1": (D,), p + ".norm1b": (D,)})
            if isinstance(m, LightningSpec):
                for n, rows in (("q", m.heads * m.dim), ("k", m.heads * m.dim), ("v", m.heads * m.vdim), ("g", m.heads * m.vdim)):
                    out[f"{q}.{n}"] = (rows, D)
                out.update({q + ".o": (D, m.heads * m.vdim), q + ".norm": (m.heads * m.vdim,)})
            elif isinstance(m, WindowSpec):
                out.update({q + ".q": (m.heads * m.dim, D), q + ".q.b": (m.heads * m.dim,), q + ".k": (m.kv_heads * m.dim, D),
                            q + ".k.b": (m.kv_heads * m.dim,), q + ".sink": (m.heads,), q + ".g": (m.heads, D),
                            q + ".o": (D, m.heads * m.dim)})
            else:
                out.update({q + ".dq": (m.q_rank, D), q + ".dq.norm": (m.q_rank,),
                            q + ".uq": (m.heads * (m.dim + m.rot_dim), m.q_rank), q + ".dkv": (m.row, D),
                            q + ".dkv.norm": (m.kv_rank,), q + ".uk": (m.heads * m.dim, m.kv_rank),
                            q + ".uv": (m.heads * m.vdim, m.kv_rank), q + ".g": (m.heads, D), q + ".o": (D, m.heads * m.vdim)})
            if f is not None:
                out.update({p + ".norm2": (D,), p + ".norm2b": (D,), p + ".mlp.up": (f.ff, D), p + ".mlp.down": (D, f.ff)})
        return out

    def _random_init(self, seed: int) -> None:
        g = torch.Generator(device=self.dev).manual_seed(seed)
        raw = {}
        for name, shape in self._tensor_names().items():
            leaf = name.rsplit(".", 1)[-1]
            t = torch.randn(*shape, generator=g, device=self.dev, dtype=torch.float32)
            if leaf == "b":
                t = 0.1 * t
            elif name.endswith((".dq.norm", ".dkv.norm", ".mix.norm")):
                t = 1.0 + 0.1 * t                    # plain norm weights
            elif leaf == "sink":
                pass
            elif len(shape) == 1:
                t = 0.1 * t                          # the layer norms' weights are stored around zero
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
        """Matrices and projection biases in the activation type, parameter vectors in fp32."""
        for k, t in raw.items():
            proj_bias = k.endswith((".q.b", ".k.b"))                 # added inside the fused projection
            self.w[k] = t.to(torch.float32 if t.dim() == 1 and not proj_bias else self.dtype).contiguous()

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
        """Per layer with tensors of its own: ONE projection matrix for everything that reads the mixer's input (lightning:
        q k v | gate; attention: q k | gate, the biases as one vector; latent: query latent | gate | key/value latent),
        the up-projections per head, the layer norms' weights as 1 + w, the logit factor inside the final norm's weight."""
        w, c, D = self.w, self.cfg, self.cfg.hidden
        pop = w.pop
        for i, L in enumerate(c.layer_specs):
            if L.weights != i:
                continue
            p, m, q = f"l{i}", L.mixer, f"l{i}.mix"
            for n in ("norm1", "norm1b") + (("norm2", "norm2b") if L.mlp is not None else ()):
                w[f"{p}.{n}"] = (1.0 + w[f"{p}.{n}"]).contiguous()
            if isinstance(m, LightningSpec):
                w[p + ".wproj"] = self._stack(i, [("qkv", [pop(q + ".q"), pop(q + ".k"), pop(q + ".v")]), ("g", [pop(q + ".g")])], D)
                w[q + ".decay"] = torch.tensor(m.decay, dtype=torch.float32, device=self.dev)
            elif isinstance(m, WindowSpec):
                bias = torch.cat([pop(q + ".q.b"), pop(q + ".k.b")])
                w[p + ".wproj"] = self._stack(i, [("qk", [pop(q + ".q"), pop(q + ".k")]), ("g", [pop(q + ".g")])], D)
                full = torch.zeros(w[p + ".wproj"].shape[0], dtype=self.dtype, device=self.dev)
                full[:bias.shape[0]] = bias
                w[p + ".bproj"] = full
            else:
                w[p + ".wproj"] = self._stack(i, [("dq", [pop(q + ".dq")]), ("g", [pop(q + ".g")]), ("dkv", [pop(q + ".dkv")])], D)
                w[q + ".uk"] = w[q + ".uk"].view(m.heads, m.dim, m.kv_rank)                                      # q_h -> latent space
                w[q + ".uv"] = w[q + ".uv"].view(m.heads, m.vdim, m.kv_rank).transpose(1, 2).contiguous()        # [H, R, dv]
        w["final.norm"] = ((1.0 + w["final.norm"]) * c.logit_scale).contiguous()

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.w.values())

    # ------------------------------------------------------------------ caches and state
    def alloc_cache(self, num_blocks: int) -> None:
        """Per attention layer a K pool (rotated keys) and a V pool (the keys as projected), [num_blocks, G, bs, dk]; per
        latent layer one pool [num_blocks, bs, kv_rank + rot_dim].  A layer that uses another layer's tensors has pools of
        its own."""
        self.num_blocks = int(num_blocks)
        self.k_cache.clear(), self.v_cache.clear(), self.latent_cache.clear()
        for i, L in enumerate(self.cfg.layer_specs):
            m = L.mixer
            if isinstance(m, WindowSpec):
                self.k_cache[i] = torch.zeros(num_blocks, m.kv_heads, self.bs, m.dim, dtype=self.dtype, device=self.dev)
                self.v_cache[i] = torch.zeros(num_blocks, m.kv_heads, self.bs, m.dim, dtype=self.dtype, device=self.dev)
            elif isinstance(m, LatentSpec):
                self.latent_cache[i] = torch.zeros(num_blocks, self.bs, m.row, dtype=self.dtype, device=self.dev)

    def alloc_state(self, max_num_seqs: int) -> None:
        """One fp32 matrix state [H, dk, dv] per live sequence and lightning layer.  Slots are never cleared: a sequence
        that starts at position 0 ignores their contents."""
        self.max_num_seqs = int(max_num_seqs)
        self.state.clear()
        for i, L in enumerate(self.cfg.layer_specs):
            m = L.mixer
            if isinstance(m, LightningSpec):
                self.state[i] = torch.zeros(max_num_seqs, m.heads, m.dim, m.vdim, dtype=torch.float32, device=self.dev)

    def prepare_decode(self, max_batch: int, max_nb: int) -> None:
        """Static index tensors of the decode-only batch (one row per sequence)."""
        if self._arange.shape[0] < max_batch + 1:
            self._arange = torch.arange(max_batch + 1, dtype=torch.int32, device=self.dev)

    def decode_schedule(self, seq_lens_host) -> int:
        return 0

    # ------------------------------------------------------------------ forward
    def _lightning(self, li: int, p: str, m: LightningSpec, h: torch.Tensor, batch: ops.SeqBatch) -> torch.Tensor:
        w, cols = self.w, self.cols[int(p[1:])]
        H, dk, dv = m.heads, m.dim, m.vdim
        T = h.shape[0]
        proj = torch.nn.functional.linear(h, w[p + ".wproj"])                  # [T, q k v | gate]
        qkv, _, decay = ops.recur_prep(proj, H, H, dk, dv, batch, conv_silu=True, decay_mode=ops.DECAY_HEAD_CONST,
                                       decay_bias=w[p + ".mix.decay"])
        o = ops.channel_scan(qkv, None, decay, H, H, dk, dv, batch, self.state[li], delta=False)
        g = cols["g"]
        out = ops.gated_head_norm(o.view(T, 1, H * dv), proj[:, g:g + H * dv], w[p + ".mix.norm"], self.cfg.eps, ops.GATE_SIGMOID)
        return torch.nn.functional.linear(out, w[p + ".mix.o"])

    def _window(self, li: int, p: str, m: WindowSpec, h: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                batch: ops.SeqBatch) -> torch.Tensor:
        w, cols = self.w, self.cols[int(p[1:])]
        H, G, dk = m.heads, m.kv_heads, m.dim
        T = h.shape[0]
        proj = torch.nn.functional.linear(h, w[p + ".wproj"], w[p + ".bproj"])      # [T, q k | gate]
        q = ops.qk_rope_cache(proj, H, G, dk, dk, positions, self.rot.get((m.rot_dims, m.rot_base)), m.rot_dims, slots,
                              self.k_cache[li], self.v_cache[li], v_from_k=True)
        g = cols["g"]
        o = ops.chunk_attention(q, self.k_cache[li], self.v_cache[li], batch, m.scale, window=m.window, keep_first=m.keep_first,
                                sink=1.0, sink_logits=w[p + ".mix.sink"], gate=proj[:, g:g + H])
        return torch.nn.functional.linear(o.view(T, H * dk), w[p + ".mix.o"])

    def _prompt_plan(self, prefill):
        """(rows N, cu_k, k_lo) of the pool rows the step's prompt portions see from position 0 on (the latent layers are
        causal, and each has a pool of its own with the same rows), or None: every row stays in the latent space."""
        if prefill is None or self.dtype != torch.bfloat16 or prefill.total_tokens < PROMPT_PER_HEAD_MIN_ROWS \
                or prefill.q_lens_host is None or prefill.kv_lens_host is None or not self.latent_cache:
            return None
        return ops.latent_prompt_plan(prefill.q_lens_host, prefill.kv_lens_host, 0,
                                      PROMPT_PER_HEAD_MAX_CONTEXT * prefill.total_tokens, self.dev)

    def _latent(self, li: int, p: str, m: LatentSpec, h: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                batch: ops.SeqBatch, n_decode: int = 0, prefill=None, plan=None) -> torch.Tensor:
        w, cols = self.w, self.cols[int(p[1:])]
        H, dn, dr, dv, R = m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank
        T = h.shape[0]
        proj = torch.nn.functional.linear(h, w[p + ".wproj"])                  # [T, query latent | gate | R + dr]
        cq = ops.row_norm(proj[:, :m.q_rank], w[p + ".mix.dq.norm"], self.cfg.eps)
        qh = torch.nn.functional.linear(cq, w[p + ".mix.uq"]).view(T, H, dn + dr)
        cache = self.latent_cache[li]
        qa = ops.latent_prep(qh.view(T, H * (dn + dr)), H, dn, dr, m.rot_dims, R, 0, cols["dkv"], w[p + ".mix.dkv.norm"],
                             self.cfg.eps, positions, self._rot_table(m), slots, cache, kv=proj)
        g = cols["g"]
        gate = proj[:, g:g + H]
        ov = torch.empty(T, H, dv, dtype=h.dtype, device=h.device)
        if plan is not None and not (ops.window_attention_ok(self.dtype, dn, dr, dv) and m.row % 8 == 0):
            plan = None
        nl = T if plan is None else n_decode            # rows that stay in the latent space
        if nl:
            # the unrotated part of every query head, carried into the latent space: qa[:, h, :R] = q_h W_uk[h]
            torch.bmm(qh[:nl, :, :dn].transpose(0, 1), w[p + ".mix.uk"], out=qa[:nl, :, :R].transpose(0, 1))
            lb = batch if plan is None else ops.SeqBatch(batch.cu_q[:nl + 1], batch.ctx_start[:nl], batch.block_tables[:nl], None, nl, nl)
            o = ops.latent_attention(qa[:nl], cache, lb, R, m.scale, 0, gate=gate[:nl])
            torch.bmm(o.transpose(0, 1), w[p + ".mix.uv"], out=ov[:nl].transpose(0, 1))   # head outputs = W_uv[h] (sum_j p_j c_j)
        if plan is not None:
            # long prompt portions: keys and values per head, rebuilt over the pool rows the portions see
            N, cu_k, k_lo = plan
            npf = len(prefill.q_lens_host)
            lat = ops.latent_gather(cache, prefill.block_tables, cu_k, k_lo, npf, N)
            kn = torch.nn.functional.linear(lat[:, :R], w[p + ".mix.uk"].view(H * dn, R)).view(N, H, dn)
            v = torch.empty(N, H, dv, dtype=h.dtype, device=h.device)
            torch.bmm(lat[:, :R].unsqueeze(0).expand(H, N, R), w[p + ".mix.uv"], out=v.transpose(0, 1))
            ov[nl:] = ops.window_attention(qh[nl:, :, :dn], qa[nl:, :, R:], kn, lat[:, R:], v, prefill.cu_q, prefill.ctx_start,
                                           cu_k, k_lo, npf, m.scale, 0, gate=gate[nl:])
        return torch.nn.functional.linear(ov.view(T, H * dv), w[p + ".mix.o"])

    def _rot_table(self, m) -> torch.Tensor:
        t = self.rot.get((m.rot_dims, m.rot_base))
        if t is None:                                # nothing turns: the kernels still take a table
            t = self.rot[(m.rot_dims, m.rot_base)] = torch.zeros(self.max_position, 0, dtype=torch.float32, device=self.dev)
        return t

    def _mixer(self, li: int, h, positions, slots, batch, n_decode=0, prefill=None, plan=None) -> torch.Tensor:
        L = self.cfg.layer_specs[li]
        p, m = f"l{L.weights}", L.mixer
        if isinstance(m, LightningSpec):
            return self._lightning(li, p, m, h, batch)
        if isinstance(m, WindowSpec):
            return self._window(li, p, m, h, positions, slots, batch)
        return self._latent(li, p, m, h, positions, slots, batch, n_decode, prefill, plan)

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
        if self.state:
            if n_decode and dec_state_slots is None:
                raise ValueError("decode rows need their state slots")
            if prefill is not None and prefill.total_tokens and prefill.state_slots is None:
                raise ValueError("prompt chunks need their state slots")
        batch = ops.step_batch(self._arange, n_decode, dec_block_tables, dec_seq_lens, dec_state_slots, prefill)
        plan = self._prompt_plan(prefill)
        T, D = tokens.shape[0], c.hidden
        rms = ops.NORM_RMS
        x = ops.embed_streams(w["embed"], tokens, 1, c.embed_scale).view(T, D)       # the fp32 residual
        n = len(c.layer_specs)
        h = ops.sandwich_norm(x, pre_w=w[f"l{c.layer_specs[0].weights}.norm1"], eps=c.eps, norm_kind=rms, h_dtype=self.dtype)
        for li in range(n):
            L = c.layer_specs[li]
            p = f"l{L.weights}"
            y = self._mixer(li, h, positions, slots, batch, n_decode, prefill, plan)
            post = w[p + ".norm1b"]
            if L.mlp is not None:
                h = ops.sandwich_norm(x, y, post, None, w[p + ".norm2"], eps=c.eps, norm_kind=rms, h_dtype=self.dtype)
                y = torch.nn.functional.linear(ops.relu_sq(torch.nn.functional.linear(h, w[p + ".mlp.up"])), w[p + ".mlp.down"])
                post = w[p + ".norm2b"]
            if li + 1 < n:
                nxt = w[f"l{c.layer_specs[li + 1].weights}.norm1"]
                h = ops.sandwich_norm(x, y, post, None, nxt, eps=c.eps, norm_kind=rms, h_dtype=self.dtype)
            else:
                ops.sandwich_norm(x, y, post, eps=c.eps, norm_kind=rms)
            if self.capture is not None:
                self.capture.append(x.clone())
        if sample_rows is not None:
            x = x.index_select(0, sample_rows).contiguous()
        h = ops.sandwich_norm(x, pre_w=w["final.norm"], eps=c.eps, norm_kind=rms, h_dtype=self.dtype)    # carries the logit factor
        return torch.nn.functional.linear(h, w["head"])
