"""Vepivik as an architecture of this engine: a pre-norm decoder whose layers have one of two windowed attention
mixers and a routed feed-forward.

* ``attention``         grouped-query softmax attention without positions in its scores, keys of size ``dim`` and
                        values of size ``vdim``, over a sliding window of ``mask.size`` positions;
* ``latent_attention``  attention over a normed latent of ``kv_rank`` sizes per token and a rotated key part of
                        ``rot_dim`` sizes shared by all heads (interleaved pairs, YaRN-interpolated frequencies),
                        the same kind of window, and a sigmoid gate on the heads' output.  A layer with ``kv_from: j``
                        has no latent of its own and reads the rows layer j cached.

Every layer's feed-forward is a mixture of experts (softmax router, the ``top`` largest scores renormalised, experts
with a squared relu, optionally a shared expert), or none.  Token rows are scaled as they enter the stream and the
output matrix is the embedding table itself.  ``config.json`` gives every size and constant; like every
architecture here the model is described as data.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from yalis_b200.config.registry import ConfigError, register_architecture
from yalis_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE_NAME = "Vepivik"
MAX_POSITION = 1 << 20          # nothing in the design bounds a sequence; block tables are sized by the cache pool
LAYER_TYPES = ("attention", "latent_attention")
RENORM_EPS = 1e-20              # added to the sum of the chosen experts' scores


@dataclass(frozen=True)
class VepivikConfig:
    width: int
    vocab: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[Mapping[str, Any], ...]     # validated copies of the config's layer entries

    @property
    def architecture(self) -> str:
        return ARCHITECTURE_NAME


def _int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = d.get(key) if isinstance(d, Mapping) else None
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{where}: `{key}` must be a positive integer, got {v!r}")
    return v


def _num(d: Mapping[str, Any], key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, Mapping) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{where}: `{key}` must be a number, got {v!r}")
    return float(v)


def _window(m: Mapping[str, Any], where: str) -> Optional[int]:
    mask = m.get("mask")
    if mask is None:
        return None
    return _int(mask, "size", where + ".mask")


def _rot(m: Mapping[str, Any], part: int, where: str) -> Optional[Dict[str, Any]]:
    rot = m.get("rot")
    if rot is None:
        return None
    where += ".rot"
    dims, base = _int(rot, "dims", where), _num(rot, "base", where)
    if dims % 2 or dims > part or base <= 1.0:
        raise ConfigError(f"{where}: dims {dims} must be even and at most {part}, base above 1")
    out: Dict[str, Any] = {"dims": dims, "base": base, "scaling": None}
    sc = rot.get("scaling")
    if sc is not None:
        out["scaling"] = {k: _num(sc, k, where + ".scaling") for k in ("factor", "original", "fast", "slow")}
        if min(out["scaling"].values()) <= 0:
            raise ConfigError(f"{where}.scaling: factor, original, fast and slow must be positive")
    return out


def _check_mlp(mlp, where: str):
    if mlp is None:
        return None
    if not isinstance(mlp, Mapping) or mlp.get("kind") != "moe":
        raise ConfigError(f"{where}: mlp kind {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r} is not supported (moe, or null)")
    out = {"kind": "moe", "expert": {"ff": _int(mlp.get("expert"), "ff", where + ".expert")},
           "router": {"experts": _int(mlp.get("router"), "experts", where + ".router"),
                      "top": _int(mlp.get("router"), "top", where + ".router")}}
    if out["router"]["top"] > out["router"]["experts"]:
        raise ConfigError(f"{where}.router: top {out['router']['top']} is more than the {out['router']['experts']} experts")
    if mlp.get("shared") is not None:
        out["shared"] = {"ff": _int(mlp["shared"], "ff", where + ".shared")}
    return out


def _check_layer(i: int, layer: Mapping[str, Any], n_layers: int) -> Dict[str, Any]:
    where = f"layers[{i}]"
    kind = layer.get("type") if isinstance(layer, Mapping) else None
    if kind not in LAYER_TYPES:
        raise ConfigError(f"{where}: type {kind!r} is not one of {', '.join(LAYER_TYPES)}")
    m = layer.get("mixer")
    if not isinstance(m, Mapping):
        raise ConfigError(f"{where}: `mixer` must be an object")
    if kind == "attention":
        mixer: Dict[str, Any] = {k: _int(m, k, where) for k in ("heads", "kv_heads", "dim", "vdim")}
        if mixer["heads"] % mixer["kv_heads"]:
            raise ConfigError(f"{where}: heads {mixer['heads']} is not a multiple of kv_heads {mixer['kv_heads']}")
    else:
        mixer = {k: _int(m, k, where) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank")}
        mixer["rot"] = _rot(m, mixer["rot_dim"], where)
        if m.get("kv_from") is not None:
            j = m["kv_from"]
            if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < i:
                raise ConfigError(f"{where}: kv_from {j!r} must name an earlier layer")
            mixer["kv_from"] = j
    mixer["scale"] = _num(m, "scale", where)
    window = _window(m, where)
    if window is not None:
        mixer["mask"] = {"size": window}
    return {"type": kind, "mixer": mixer, "mlp": _check_mlp(layer.get("mlp"), where + ".mlp")}


class VepivikArchitecture:
    name = ARCHITECTURE_NAME

    @staticmethod
    def parse_config(raw: Dict[str, Any]) -> VepivikConfig:
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json lacks `layers`")
        eps = _num(raw.get("norm"), "eps", "norm")
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        checked = tuple(_check_layer(i, l, len(layers)) for i, l in enumerate(layers))
        for i, layer in enumerate(checked):
            j = layer["mixer"].get("kv_from")
            if j is None:
                continue
            src, m = checked[j], layer["mixer"]
            if src["type"] != "latent_attention" or src["mixer"].get("kv_from") is not None:
                raise ConfigError(f"layers[{i}]: kv_from {j} must name a latent_attention layer with a latent of its own")
            if any(src["mixer"][k] != m[k] for k in ("kv_rank", "rot_dim", "rot")):
                raise ConfigError(f"layers[{i}]: kv_rank, rot_dim and rot must equal those of layer {j}, whose rows it reads")
        scale = _num(raw.get("embedding"), "scale", "embedding") if raw.get("embedding") is not None else 1.0
        return VepivikConfig(width=_int(raw, "width", "config"), vocab=_int(raw, "vocab", "config"), norm_eps=eps,
                             embedding_scale=scale, layers=checked)

    @staticmethod
    def config_to_dict(c: VepivikConfig) -> Dict[str, Any]:
        layers = copy.deepcopy([dict(l) for l in c.layers])
        for layer in layers:
            m = layer["mixer"]
            if layer["type"] == "latent_attention" and m.get("rot") is not None and m["rot"].get("scaling") is None:
                m["rot"] = {k: v for k, v in m["rot"].items() if k != "scaling"}
        return {"architecture": ARCHITECTURE_NAME, "embedding": {"scale": c.embedding_scale}, "layers": layers,
                "norm": {"eps": c.norm_eps}, "vocab": c.vocab, "width": c.width}

    @staticmethod
    def _window_of(layer: Mapping[str, Any]) -> Optional[int]:
        mask = layer["mixer"].get("mask")
        return None if mask is None else mask["size"]

    @classmethod
    def _kept(cls, c: VepivikConfig, owner: int) -> Optional[int]:
        """How many positions back the rows of latent layer ``owner`` must be kept: the widest window among the
        layer itself and the layers that read its rows (None: for ever)."""
        windows = [cls._window_of(l) for i, l in enumerate(c.layers)
                   if i == owner or (l["type"] == "latent_attention" and l["mixer"].get("kv_from") == owner)]
        return None if any(w is None for w in windows) else max(windows)

    @classmethod
    def _layer(cls, c: VepivikConfig, i: int, layer: Mapping[str, Any]) -> LayerSpec:
        kind, m = layer["type"], layer["mixer"]
        names = {"norm_1.weight": "norm1"}
        window = cls._window_of(layer)
        if kind == "attention":
            mixer = PartSpec("general_attention", {
                "hidden_size": c.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "v_head_dim": m["vdim"], "bias": False, "qk_norm_eps": None, "rotary": None, "scale": m["scale"],
                "softcap": None, "sink": False, "window": window, "out_scale": 1.0})
            names.update({f"mixer.{p}_proj": f"mix.{p}" for p in ("q", "k", "v", "o")})
        else:
            own = m.get("kv_from") is None
            rotary = None
            if m["rot"] is not None:
                sc = m["rot"]["scaling"]
                rotary = {"head_dim": m["rot"]["dims"], "theta": m["rot"]["base"], "layout": "interleaved", "exact_powers": True,
                          "scaling": None if sc is None else {"kind": "yarn", **sc}}
            mixer = PartSpec("latent_attention", {
                "hidden_size": c.width, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
                "v_head_dim": m["vdim"], "kv_rank": m["kv_rank"], "rotary": rotary, "scale": m["scale"], "window": window,
                "cache_window": cls._kept(c, i if own else m["kv_from"]), "norm_eps": c.norm_eps, "gate": True,
                "own_latent": own})
            names.update({"mixer.q_proj": "mix.q", "mixer.uk_proj": "mix.uk", "mixer.uv_proj": "mix.uv",
                          "mixer.g_proj": "mix.g", "mixer.o_proj": "mix.o"})
            if own:
                names.update({"mixer.dkv_proj": "mix.dkv", "mixer.dkv_norm": "mix.dkv.norm"})
        parts = {"norm_1": PartSpec("rms_norm", {"size": c.width, "eps": c.norm_eps}), "mixer": mixer}
        mlp = layer["mlp"]
        if mlp is not None:
            shared = mlp.get("shared")
            parts["norm_2"] = PartSpec("rms_norm", {"size": c.width, "eps": c.norm_eps})
            parts["feed_forward"] = PartSpec("routed_experts", {
                "hidden_size": c.width, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                "expert_size": mlp["expert"]["ff"], "activation": "relu2",
                "shared_size": None if shared is None else shared["ff"], "renorm_eps": RENORM_EPS})
            names.update({"norm_2.weight": "norm2", "feed_forward.router": "mlp.router"})
            for e in range(mlp["router"]["experts"]):
                names[f"feed_forward.expert_{e}_up"] = f"mlp.e{e}.up"
                names[f"feed_forward.expert_{e}_down"] = f"mlp.e{e}.down"
            if shared is not None:
                names.update({"feed_forward.shared_up": "mlp.shared.up", "feed_forward.shared_down": "mlp.shared.down"})
        return LayerSpec(block=PartSpec("pre_norm_residual"), parts=parts, weight_prefix=f"l{i}.", weight_names=names)

    @classmethod
    def model_spec(cls, c: VepivikConfig) -> ModelSpec:
        # a layer that reads another layer's rows is a schedule entry that reads that entry's cache
        schedule = tuple(ScheduleEntry(i, cache_of=layer["mixer"].get("kv_from")) for i, layer in enumerate(c.layers))
        return ModelSpec(
            architecture=ARCHITECTURE_NAME, hidden_size=c.width, vocab_size=c.vocab, max_position=MAX_POSITION,
            layers=tuple(cls._layer(c, i, layer) for i, layer in enumerate(c.layers)), schedule=schedule,
            final_norm=PartSpec("rms_norm", {"size": c.width, "eps": c.norm_eps}),
            embedding_name="embed", head_name=None, final_norm_names={"weight": "final.norm"},
            embedding_scale=c.embedding_scale)


register_architecture(ARCHITECTURE_NAME, VepivikArchitecture, replace=True)
