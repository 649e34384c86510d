"""Gatolix decoder on the b200attn ops: layers with a layer norm (weight and bias) before AND after every sublayer around
one fp32 residual; the sequence mixer is sliding-window attention over a low-rank latent that all heads share (plus one
shared rotated key part, interleaved rotary pairs with YaRN frequency scaling), with a sigmoid gate per head; a layer
may read another layer's latent pool instead of projecting its own; the feed-forward is dense (squared ReLU) or a
routed mixture of bounded gated experts whose choice adds a correction to the softmax scores; the logits are soft-capped.

The model plugs into the same engine as LlamaModel and KofadraModel (b200attn.engine.LLMEngine): a paged pool per layer
that owns a down-projection, addressed through the scheduler's block tables and slot mapping, one forward over
[decode rows | prompt chunks], logits for the sampled rows.  Projections, the per-head up-projections (batched) and the
vocabulary head are library GEMMs (torch -> cuBLAS); everything between them is this repo's kernels
(csrc/post_norm.cu, latent_attention.cu, moe.cu).  There is no CPU path.

Attention runs in the latent space: W_uk is applied to the query (one batched product per step) so that scores are
taken against the cached rows directly, and W_uv is applied to the attention output; keys and values per head are not
materialised for decode rows and short portions.  A step with many prompt rows (bf16) rebuilds them per head for the
pool rows its portions can see, which costs a third of the multiplications per (query, key) pair.

Every size, the layer order and every constant come from the checkpoint's config.json (`architecture: "Gatolix"`);
weights from its *.safetensors, or random from a seed.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Optional, Tuple, Union

import torch

from . import ops

ARCHITECTURE = "Gatolix"
GLU_ALPHA = 1.702          # the design fixes the slope of the experts' gate sigmoid
# A step with at least this many prompt rows rebuilds keys and values per head for them (bf16): (dim + rot_dim + vdim)
# multiplications per (query, key, head) instead of (2 kv_rank + rot_dim) in the latent space, for two more GEMMs per layer
# over the rows the portions can see.  Decode rows and short portions stay in the latent space.
PROMPT_PER_HEAD_MIN_ROWS = 256
PROMPT_PER_HEAD_MAX_CONTEXT = 4      # ... unless the visible rows outnumber the prompt rows by more than this factor


@dataclass
class LatentSpec:
    heads: int
    dim: int                   # per-head unrotated query / key size
    rot_dim: int               # per-head rotated query size = size of the shared rotated key part
    vdim: int                  # per-head value size
    kv_rank: int               # latent size
    scale: float               # score scale
    window: int = 0            # a query attends to its own position and the window - 1 before it (0: plain causal)
    rot_dims: int = 0          # how many entries of the rotated part turn (the rest pass)
    rot_base: float = 10000.0
    rot_scaling: Optional[dict] = None     # {factor, original, fast, slow}
    kv_from: Optional[int] = None          # the layer whose latent pool this layer reads

    @property
    def row(self) -> int:
        return self.kv_rank + self.rot_dim

    @property
    def rot_key(self) -> tuple:
        s = self.rot_scaling
        return (self.rot_dims, self.rot_base, None if not s else tuple(sorted((k, float(v)) for k, v in s.items())))


@dataclass
class DenseSpec:
    ff: int


@dataclass
class ExpertsSpec:
    experts: int
    top: int
    ff: int
    limit: float


@dataclass
class LayerSpec:
    mixer: LatentSpec
    mlp: Union[None, DenseSpec, ExpertsSpec]


@dataclass
class GatolixConfig:
    name: str
    vocab: int
    hidden: int
    layer_specs: List[LayerSpec]
    eps: float = 1e-6
    logit_softcap: float = 0.0             # 0: none
    max_position: int = 1 << 20            # the rotary table is built for the engine's max_model_len
    family: str = "gatolix"

    @property
    def layers(self) -> int:
        return len(self.layer_specs)

    @property
    def params(self) -> int:
        D = self.hidden
        n = 2 * self.vocab * D + 2 * D
        for L in self.layer_specs:
            m = L.mixer
            n += D * (m.heads * (m.dim + m.rot_dim) + m.heads) + m.kv_rank * m.heads * (m.dim + m.vdim) + m.heads * m.vdim * D
            n += 4 * D
            if m.kv_from is None:
                n += D * m.row + m.kv_rank
            if isinstance(L.mlp, DenseSpec):
                n += 2 * D * L.mlp.ff + 4 * D
            elif L.mlp is not None:
                n += L.mlp.experts * (3 * L.mlp.ff * D + D + 1) + 4 * D
        return n

    def kv_bytes_per_token(self, kv_elem_bytes: int = 2, tp: int = 1) -> int:
        return sum(L.mixer.row * kv_elem_bytes for L in self.layer_specs if L.mixer.kv_from is None)

    def state_bytes_per_seq(self, elem_bytes: int = 2) -> int:
        return 0                                     # attention only: nothing is kept per sequence besides the pools

    def activation_bytes(self, tokens: int, seqs: int, elem_bytes: int = 2) -> int:
        wide = max([self.hidden] + [m.heads * (m.dim + m.rot_dim + 1 + 2 * m.row + m.vdim) + m.row
                                    for m in (L.mixer for L in self.layer_specs)]
                   + [L.mlp.ff * 2 for L in self.layer_specs if isinstance(L.mlp, DenseSpec)])
        moe = max([0] + [L.mlp.top * (3 * L.mlp.ff * elem_bytes + self.hidden * 4) for L in self.layer_specs
                         if isinstance(L.mlp, ExpertsSpec)])
        return tokens * (self.hidden * 8 + 2 * wide * elem_bytes + 2 * moe) + seqs * self.vocab * 8 + (1 << 28)

    def build_model(self, device, **kw):
        return GatolixModel(self, device, **kw)


def config_from_dict(c: dict, name: str = ARCHITECTURE) -> GatolixConfig:
    """config.json -> GatolixConfig.  Keys: vocab, width, norm.eps, logit_softcap, layers [{type: latent_attention,
    mixer {heads, dim, rot_dim, vdim, kv_rank, scale, mask.size, rot {base, dims, scaling {factor, original, fast, slow}},
    kv_from}, mlp null | {kind: dense, ff} | {kind: moe, expert {ff, limit}, router {experts, top}}}]."""
    specs: List[LayerSpec] = []
    for i, L in enumerate(c["layers"]):
        if L["type"] != "latent_attention":
            raise ValueError(f"layer {i}: unknown mixer type {L['type']!r}")
        m = L["mixer"]
        rot = m.get("rot") or {}
        rot_dim = int(m["rot_dim"])
        spec = LatentSpec(heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=rot_dim, vdim=int(m["vdim"]),
                          kv_rank=int(m["kv_rank"]), scale=float(m["scale"]),
                          window=int((m.get("mask") or {}).get("size") or 0), rot_dims=int(rot.get("dims", rot_dim)),
                          rot_base=float(rot.get("base", 10000.0)), rot_scaling=rot.get("scaling") or None,
                          kv_from=None if m.get("kv_from") is None else int(m["kv_from"]))
        if spec.rot_dims % 2 or not 0 <= spec.rot_dims <= rot_dim:
            raise ValueError(f"layer {i}: rot.dims {spec.rot_dims} must be even and at most rot_dim {rot_dim}")
        if spec.kv_from is not None:
            j = spec.kv_from
            if not 0 <= j < i or specs[j].mixer.kv_from is not None:
                raise ValueError(f"layer {i}: kv_from {j} must name an earlier layer with a down-projection of its own")
            o = specs[j].mixer
            if (o.kv_rank, o.rot_dim, o.rot_key) != (spec.kv_rank, spec.rot_dim, spec.rot_key):
                raise ValueError(f"layer {i}: latent size and rotation differ from layer {j}, whose pool it reads")
        f = L.get("mlp")
        mlp: Union[None, DenseSpec, ExpertsSpec] = None
        if f:
            kind = f.get("kind")
            if kind == "dense":
                mlp = DenseSpec(int(f["ff"]))
            elif kind == "moe":
                mlp = ExpertsSpec(int(f["router"]["experts"]), int(f["router"]["top"]), int(f["expert"]["ff"]),
                                  float(f["expert"]["limit"]))
                if not 1 <= mlp.top <= mlp.experts:
                    raise ValueError(f"layer {i}: router picks {mlp.top} of {mlp.experts} experts")
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {kind!r}")
        specs.append(LayerSpec(spec, mlp))
    return GatolixConfig(name=name, vocab=int(c["vocab"]), hidden=int(c["width"]), layer_specs=specs,
                         eps=float((c.get("norm") or {}).get("eps", 1e-6)), logit_softcap=float(c.get("logit_softcap") or 0.0))


def config_from_dir(path: Path) -> GatolixConfig:
    return config_from_dict(json.loads((Path(path) / "config.json").read_text()), name=Path(path).name)


def bench_config(hidden: int, layers: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, ff: int,
                 experts: int, top: int, vocab: int, window: int = 1024, share_every: int = 2,
                 name: str = "gatolix-bench") -> GatolixConfig:
    """A model-sized geometry for benchmarks: layer 0 dense, the rest routed; every `share_every`-th layer owns a latent
    pool and the layers after it read it."""
    specs = []
    scaling = {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}
    for i in range(layers):
        owner = i - i % max(share_every, 1)
        m = LatentSpec(heads, dim, rot_dim, vdim, kv_rank, (dim + rot_dim) ** -0.5, window, rot_dim, 10000.0, scaling,
                       None if owner == i else owner)
        specs.append(LayerSpec(m, DenseSpec(ff * top) if i == 0 else ExpertsSpec(experts, top, ff, 7.0)))
    return GatolixConfig(name, vocab, hidden, specs, logit_softcap=30.0)


class GatolixModel:
    """Weights + per-layer latent pools + forward over one scheduled token batch.  One instance per GPU."""

    supports_fp32 = True
    launches_per_layer = 10

    def __init__(self, cfg: GatolixConfig, device: torch.device, num_blocks: int, block_size: int = 16, seed: int = 0,
                 weights_dir: Optional[Path] = None, max_position: Optional[int] = None,
                 kv_dtype: torch.dtype = torch.bfloat16, tp=None, dtype: torch.dtype = torch.bfloat16,
                 max_num_seqs: int = 1):
        if device.type != "cuda":
            raise ValueError("GatolixModel needs a CUDA device (b200attn has no CPU path)")
        if tp is not None and tp.size > 1:
            raise ValueError("Gatolix runs on one GPU per replica: tensor_parallel_size must be 1")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {dtype}: bfloat16 or float32")
        if kv_dtype not in (torch.bfloat16, dtype):
            raise ValueError("Gatolix keeps its latent pools in the activation type (no fp8 cache)")
        self.cfg, self.dev, self.bs, self.dtype = cfg, device, block_size, dtype
        self.tp, self.tp_size, self.tp_rank = None, 1, 0
        self.vocab_parallel = False
        self.Hq = self.Hkv = 0                      # no paged-decode schedule to plan
        self.max_position = max_position or min(cfg.max_position, 1 << 17)
        self.max_num_seqs = max_num_seqs
        self.w: Dict[str, torch.Tensor] = {}
        if weights_dir is not None and any(Path(weights_dir).glob("*.safetensors")):
            self._load(Path(weights_dir))
        else:
            self._random_init(seed)
        self._fuse()
        # one rotary table per distinct (dims, base, scaling)
        self.rot: Dict[tuple, torch.Tensor] = {}
        for L in cfg.layer_specs:
            m = L.mixer
            if m.rot_key not in self.rot:
                self.rot[m.rot_key] = ops.rotary_table(self.max_position, m.rot_dims, m.rot_base, m.rot_scaling, device)
        self.num_blocks = 0
        self.cache: Dict[int, torch.Tensor] = {}
        self.alloc_cache(num_blocks)
        self._arange = torch.arange(max_num_seqs + 1, dtype=torch.int32, device=device)
        self.capture: Optional[list] = None         # tests: set to a list to collect the residual after every layer

    # ------------------------------------------------------------------ weights
    def _tensor_names(self) -> Dict[str, Tuple[int, ...]]:
        """Name -> shape of every tensor of a checkpoint of this configuration."""
        c, D = self.cfg, self.cfg.hidden
        out = {"embed": (c.vocab, D), "final.norm": (D,), "final.norm.b": (D,), "head": (c.vocab, D)}
        for i, L in enumerate(c.layer_specs):
            p, m, f = f"l{i}", L.mixer, L.mlp
            for n in ("norm1", "norm1b") + (("norm2", "norm2b") if f is not None else ()):
                out[f"{p}.{n}"] = (D,)
                out[f"{p}.{n}.b"] = (D,)
            out[p + ".mix.q"] = (m.heads * (m.dim + m.rot_dim), D)
            if m.kv_from is None:
                out[p + ".mix.dkv"] = (m.row, D)
                out[p + ".mix.dkv.norm"] = (m.kv_rank,)
            out.update({p + ".mix.uk": (m.heads * m.dim, m.kv_rank), p + ".mix.uv": (m.heads * m.vdim, m.kv_rank),
                        p + ".mix.g": (m.heads, D), p + ".mix.o": (D, m.heads * m.vdim)})
            if isinstance(f, DenseSpec):
                out.update({p + ".mlp.up": (f.ff, D), p + ".mlp.down": (D, f.ff)})
            elif f is not None:
                for e in range(f.experts):
                    out.update({f"{p}.mlp.e{e}.gate": (f.ff, D), f"{p}.mlp.e{e}.up": (f.ff, D),
                                f"{p}.mlp.e{e}.down": (D, f.ff)})
                out.update({p + ".mlp.router": (f.experts, D), p + ".mlp.correction": (f.experts,)})
        return out

    def _random_init(self, seed: int) -> None:
        g = torch.Generator(device=self.dev).manual_seed(seed)
        raw = {}
        for name, shape in self._tensor_names().items():
            leaf = name.rsplit(".", 1)[-1]
            t = torch.randn(*shape, generator=g, device=self.dev, dtype=torch.float32)
            if leaf == "b":
                t = 0.05 * t
            elif leaf == "correction":
                t = 0.02 * t
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
        """Matrices in the activation type, parameter vectors in fp32."""
        for k, t in raw.items():
            self.w[k] = t.to(torch.float32 if t.dim() == 1 else self.dtype).contiguous()

    def _fuse(self) -> None:
        """Per layer: one projection matrix for everything that reads the mixer's input (q | gate | down-projection),
        the gate's columns padded to a multiple of eight, the up-projections per head, stacked expert matrices."""
        w, c = self.w, self.cfg
        for i, L in enumerate(c.layer_specs):
            p, m, f = f"l{i}", L.mixer, L.mlp
            g = w.pop(p + ".mix.g")
            pad = torch.zeros((-m.heads) % 8, g.shape[1], dtype=g.dtype, device=g.device)     # keeps what follows 16-byte aligned
            parts = [w.pop(p + ".mix.q"), g, pad]
            if m.kv_from is None:
                parts.append(w.pop(p + ".mix.dkv"))
            w[p + ".wproj"] = torch.cat(parts).contiguous()
            w[p + ".mix.uk"] = w[p + ".mix.uk"].view(m.heads, m.dim, m.kv_rank)                         # q_h -> latent space
            w[p + ".mix.uv"] = w[p + ".mix.uv"].view(m.heads, m.vdim, m.kv_rank).transpose(1, 2).contiguous()   # [H, R, dv]
            if isinstance(f, ExpertsSpec):
                w[f"{p}.mlp.gate_up"] = torch.stack([torch.cat([w.pop(f"{p}.mlp.e{e}.gate"), w.pop(f"{p}.mlp.e{e}.up")])
                                                     for e in range(f.experts)]).contiguous()
                w[f"{p}.mlp.down"] = torch.stack([w.pop(f"{p}.mlp.e{e}.down") for e in range(f.experts)]).contiguous()

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.w.values())

    # ------------------------------------------------------------------ caches
    def alloc_cache(self, num_blocks: int) -> None:
        """One latent pool per layer that owns a down-projection: [num_blocks, bs, kv_rank + rot_dim]."""
        self.num_blocks = int(num_blocks)
        self.cache.clear()
        for i, L in enumerate(self.cfg.layer_specs):
            if L.mixer.kv_from is None:
                self.cache[i] = torch.zeros(num_blocks, self.bs, L.mixer.row, dtype=self.dtype, device=self.dev)

    def alloc_state(self, max_num_seqs: int) -> None:
        """Nothing is kept per sequence besides the pools."""
        self.max_num_seqs = int(max_num_seqs)

    def prepare_decode(self, max_batch: int, max_nb: int) -> None:
        """Static index tensors of the decode-only batch (one row per sequence)."""
        if self._arange.shape[0] < max_batch + 1:
            self._arange = torch.arange(max_batch + 1, dtype=torch.int32, device=self.dev)

    def decode_schedule(self, seq_lens_host) -> int:
        return 0

    # ------------------------------------------------------------------ forward
    def _ln(self, name: str):
        return self.w[name], self.w[name + ".b"]

    def _prompt_plan(self, prefill) -> Optional[dict]:
        """Host-side plan of the per-head path for the step's prompt portions: owner layer -> (rows N, cu_k, k_lo) of the
        gathered pool rows, covering the widest window among the layers that read the pool.  None: the latent path."""
        if prefill is None or self.dtype != torch.bfloat16 or prefill.total_tokens < PROMPT_PER_HEAD_MIN_ROWS \
                or prefill.q_lens_host is None or prefill.kv_lens_host is None:
            return None
        specs = [L.mixer for L in self.cfg.layer_specs]
        if not all(ops.window_attention_ok(self.dtype, m.dim, m.rot_dim, m.vdim) and m.row % 8 == 0 for m in specs):
            return None
        plan = {}
        for o, mo in enumerate(specs):
            if mo.kv_from is not None:
                continue
            windows = [m.window for i, m in enumerate(specs) if i == o or m.kv_from == o]
            reach = 0 if 0 in windows else max(windows)
            one = ops.latent_prompt_plan(prefill.q_lens_host, prefill.kv_lens_host, reach,
                                         PROMPT_PER_HEAD_MAX_CONTEXT * prefill.total_tokens, self.dev)
            if one is None:
                return None
            plan[o] = one
        return plan

    def _mixer(self, li: int, h: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, batch: ops.SeqBatch,
               n_decode: int = 0, prefill=None, plan: Optional[dict] = None, gathered: Optional[dict] = None) -> torch.Tensor:
        m, w, p = self.cfg.layer_specs[li].mixer, self.w, f"l{li}"
        H, dn, dr, dv, R = m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank
        T = h.shape[0]
        proj = torch.nn.functional.linear(h, w[p + ".wproj"])                  # [T, H (dn + dr) | H, padding | R + dr]
        g_off = H * (dn + dr)
        d_off = g_off + H + (-H) % 8
        own = m.kv_from is None
        owner = li if own else m.kv_from
        cache = self.cache[owner]
        qa = ops.latent_prep(proj, H, dn, dr, m.rot_dims, R, 0, d_off if own else -1, w.get(p + ".mix.dkv.norm"),
                             self.cfg.eps, positions, self.rot[m.rot_key], slots if own else None, cache if own else None)
        qh = proj[:, :g_off].view(T, H, dn + dr)
        gate = proj[:, g_off:g_off + H]
        ov = torch.empty(T, H, dv, dtype=h.dtype, device=h.device)
        nl = T if plan is None else n_decode            # rows that stay in the latent space
        if nl:
            # the unrotated part of every query head, carried into the latent space: qa[:, h, :R] = q_h W_uk[h]
            torch.bmm(qh[:nl, :, :dn].transpose(0, 1), w[p + ".mix.uk"], out=qa[:nl, :, :R].transpose(0, 1))
            lb = batch if plan is None else ops.SeqBatch(batch.cu_q[:nl + 1], batch.ctx_start[:nl], batch.block_tables[:nl], None, nl, nl)
            o = ops.latent_attention(qa[:nl], cache, lb, R, m.scale, m.window, gate=gate[:nl])
            torch.bmm(o.transpose(0, 1), w[p + ".mix.uv"], out=ov[:nl].transpose(0, 1))   # head outputs = W_uv[h] (sum_j p_j c_j)
        if plan is not None:
            N, cu_k, k_lo = plan[owner]
            npf = len(prefill.q_lens_host)
            if owner not in gathered:                   # the owner has written this step's rows: gather once per pool
                gathered[owner] = ops.latent_gather(cache, prefill.block_tables, cu_k, k_lo, npf, N)
            lat = gathered[owner]
            kn = torch.nn.functional.linear(lat[:, :R], w[p + ".mix.uk"].view(H * dn, R)).view(N, H, dn)
            v = torch.empty(N, H, dv, dtype=h.dtype, device=h.device)
            torch.bmm(lat[:, :R].unsqueeze(0).expand(H, N, R), w[p + ".mix.uv"], out=v.transpose(0, 1))
            ov[nl:] = ops.window_attention(qh[nl:, :, :dn], qa[nl:, :, R:], kn, lat[:, R:], v, prefill.cu_q, prefill.ctx_start,
                                           cu_k, k_lo, npf, m.scale, m.window, gate=gate[nl:])
        return torch.nn.functional.linear(ov.view(T, H * dv), w[p + ".mix.o"])

    def _mlp(self, li: int, h: torch.Tensor) -> torch.Tensor:
        f, w, p = self.cfg.layer_specs[li].mlp, self.w, f"l{li}.mlp"
        if isinstance(f, DenseSpec):
            return torch.nn.functional.linear(ops.relu_sq(torch.nn.functional.linear(h, w[p + ".up"])), w[p + ".down"])
        ids, wts = ops.moe_route(h, w[p + ".router"], w[p + ".correction"], f.top, scoring=ops.ROUTE_SOFTMAX_ALL)
        gu = w[p + ".gate_up"]
        return ops.moe_experts(h, ids, wts, gu[:, :f.ff], gu[:, f.ff:], w[p + ".down"], w_gate_up=gu, glu=ops.GLU_CLAMPED,
                               glu_alpha=GLU_ALPHA, glu_limit=f.limit)

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
        batch = ops.step_batch(self._arange, n_decode, dec_block_tables, dec_seq_lens, None, prefill)
        plan = self._prompt_plan(prefill)
        gathered: Dict[int, torch.Tensor] = {}
        T, D = tokens.shape[0], c.hidden
        x = ops.embed_streams(w["embed"], tokens, 1, 1.0).view(T, D)            # the fp32 residual
        n = len(c.layer_specs)
        h = ops.sandwich_norm(x, None, None, None, *self._ln("l0.norm1"), eps=c.eps, h_dtype=self.dtype)
        for li in range(n):
            p = f"l{li}"
            y = self._mixer(li, h, positions, slots, batch, n_decode, prefill, plan, gathered)
            post = self._ln(p + ".norm1b")
            if c.layer_specs[li].mlp is not None:
                h = ops.sandwich_norm(x, y, *post, *self._ln(p + ".norm2"), eps=c.eps, h_dtype=self.dtype)
                y = self._mlp(li, h)
                post = self._ln(p + ".norm2b")
            if li + 1 < n:
                h = ops.sandwich_norm(x, y, *post, *self._ln(f"l{li + 1}.norm1"), eps=c.eps, h_dtype=self.dtype)
            else:
                ops.sandwich_norm(x, y, *post, eps=c.eps)
            if self.capture is not None:
                self.capture.append(x.clone())
        if sample_rows is not None:
            x = x.index_select(0, sample_rows).contiguous()
        h = ops.sandwich_norm(x, None, None, None, *self._ln("final.norm"), eps=c.eps, h_dtype=self.dtype)
        logits = torch.nn.functional.linear(h, w["head"])
        if c.logit_softcap > 0:
            ops.softcap_(logits, c.logit_softcap)
        return logits
