"""Tirezen as an architecture of this engine: a decoder whose layers mix three kinds of token mixer.

Every layer is a parallel block, x += mixer(norm(x)) + mlp(norm(x)), with a norm whose stored weight lies
around zero (scale 1 + w), a dense gelu feed-forward (or none), and one of

* ``retention``  a linear recurrence with a fixed decay per head over rotated q and k;
* ``delta``      the gated delta rule behind short convolutions, one decay per token and head;
* ``parallel``   softmax attention (biases, query/key norm, partial rotation, soft-capped scores, a sink in the
                 denominator) beside a delta rule whose decay has a value per key channel, added with two factors.

A range of layers may run several times in a row with the same weights (``loop``): every pass has a cache and a
state of its own, and before a pass the embedding rows (from the second pass on) and a learned vector per pass
are added to the stream.

``config.json`` gives every size and constant, with two exceptions that only tensor shapes give: the inner sizes
of the two low-rank products of the parallel mixer's right side.  ``sizes_from_tensors`` reads them from the
checkpoint's header; a configuration written by this package carries them as ``decay_rank`` and ``gate_rank``.
Like every architecture here the model is described as data: no tensor is touched in this file.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from yalis_b200.config.registry import ConfigError, register_architecture
from yalis_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, StreamInjection

ARCHITECTURE_NAME = "Tirezen"
MAX_POSITION = 1 << 20          # nothing in the design bounds a sequence; block tables are sized by the cache pool
LAYER_TYPES = ("retention", "delta", "parallel")


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class TirezenConfig:
    width: int
    vocab: int
    norm_eps: float
    layers: Tuple[Mapping[str, Any], ...]     # validated copies of the config's layer entries
    loop: Optional[Loop]

    @property
    def architecture(self) -> str:
        return ARCHITECTURE_NAME


def _int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{where}: `{key}` must be a positive integer, got {v!r}")
    return v


def _num(d: Mapping[str, Any], key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{where}: `{key}` must be a number, got {v!r}")
    return float(v)


def _rot(d: Mapping[str, Any], dim: int, where: str) -> Optional[Dict[str, Any]]:
    rot = d.get("rot")
    if rot is None:
        return None
    dims, base = _int(rot, "dims", where + ".rot"), _num(rot, "base", where + ".rot")
    if dims % 2 or dims > dim or base <= 0:
        raise ConfigError(f"{where}.rot: dims {dims} must be even and at most dim {dim}, base positive")
    return {"dims": dims, "base": base}


def _check_delta(m: Mapping[str, Any], where: str, low_rank: bool) -> Dict[str, Any]:
    out = {k: _int(m, k, where) for k in ("heads", "kv_heads", "dim", "vdim", "conv")}
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"{where}: heads {out['heads']} is not a multiple of kv_heads {out['kv_heads']}")
    if low_rank:
        for k in ("decay_rank", "gate_rank"):
            if m.get(k) is None:
                raise ConfigError(f"{where}: `{k}` is not given (a model folder gives it by the shape of its tensors)")
            out[k] = _int(m, k, where)
    return out


def _check_attention(m: Mapping[str, Any], where: str) -> Dict[str, Any]:
    out = {k: _int(m, k, where) for k in ("heads", "kv_heads", "dim", "vdim")}
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"{where}: heads {out['heads']} is not a multiple of kv_heads {out['kv_heads']}")
    out["rot"] = _rot(m, out["dim"], where)
    out["scale"] = _num(m, "scale", where)
    out["softcap"] = _num(m, "softcap", where) if m.get("softcap") is not None else None
    if out["softcap"] is not None and out["softcap"] <= 0:
        raise ConfigError(f"{where}: `softcap` must be positive")
    return out


def _check_layer(i: int, layer: Mapping[str, Any]) -> Dict[str, Any]:
    where = f"layers[{i}]"
    kind = layer.get("type")
    if kind not in LAYER_TYPES:
        raise ConfigError(f"{where}: type {kind!r} is not one of {', '.join(LAYER_TYPES)}")
    m = layer.get("mixer")
    if not isinstance(m, Mapping):
        raise ConfigError(f"{where}: `mixer` must be an object")
    if kind == "retention":
        mixer = {k: _int(m, k, where) for k in ("heads", "dim", "vdim")}
        decay = m.get("decay")
        if not isinstance(decay, (list, tuple)) or len(decay) != mixer["heads"]:
            raise ConfigError(f"{where}: `decay` must list one number per head")
        mixer["decay"] = [float(x) for x in decay]
        mixer["rot"] = _rot(m, mixer["dim"], where)
    elif kind == "delta":
        mixer = _check_delta(m, where, low_rank=False)
    else:
        for side in ("left", "right"):
            if not isinstance(m.get(side), Mapping):
                raise ConfigError(f"{where}: a parallel mixer needs `{side}`")
        mixer = {"left": _check_attention(m["left"], where + ".left"),
                 "right": _check_delta(m["right"], where + ".right", low_rank=True),
                 "left_scale": _num(m, "left_scale", where), "right_scale": _num(m, "right_scale", where)}
    mlp = layer.get("mlp")
    if mlp is not None:
        if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
            raise ConfigError(f"{where}: mlp kind {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r} is not supported (dense, or null)")
        mlp = {"kind": "dense", "ff": _int(mlp, "ff", where + ".mlp")}
    return {"type": kind, "mixer": mixer, "mlp": mlp}


class TirezenArchitecture:
    name = ARCHITECTURE_NAME

    @staticmethod
    def sizes_from_tensors(raw: Dict[str, Any], shapes: Mapping[str, Tuple[int, ...]]) -> Dict[str, Any]:
        """The configuration with the sizes that only tensor shapes give filled in."""
        raw = copy.deepcopy(raw)
        for i, layer in enumerate(raw.get("layers") or []):
            if isinstance(layer, dict) and layer.get("type") == "parallel" and isinstance(layer.get("mixer", {}).get("right"), dict):
                right = layer["mixer"]["right"]
                for key, tensor in (("decay_rank", f"l{i}.mix.right.a1"), ("gate_rank", f"l{i}.mix.right.g1")):
                    if tensor in shapes and len(shapes[tensor]) == 2:
                        right[key] = int(shapes[tensor][0])
        return raw

    @staticmethod
    def parse_config(raw: Dict[str, Any]) -> TirezenConfig:
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json lacks `layers`")
        norm = raw.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("config.json lacks `norm`")
        eps = _num(norm, "eps", "norm")
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        loop = None
        if raw.get("loop") is not None:
            lp = raw["loop"]
            start, stop, times = lp.get("start"), lp.get("stop"), _int(lp, "times", "loop")
            if not all(isinstance(v, int) and not isinstance(v, bool) for v in (start, stop)) or not 0 <= start <= stop <= len(layers):
                raise ConfigError(f"loop: start {start!r} and stop {stop!r} must satisfy 0 <= start <= stop <= {len(layers)}")
            loop = Loop(start, stop, times)
        return TirezenConfig(width=_int(raw, "width", "config"), vocab=_int(raw, "vocab", "config"), norm_eps=eps,
                             layers=tuple(_check_layer(i, l) for i, l in enumerate(layers)), loop=loop)

    @staticmethod
    def config_to_dict(c: TirezenConfig) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": ARCHITECTURE_NAME, "layers": copy.deepcopy(list(c.layers)),
                             "norm": {"eps": c.norm_eps}, "vocab": c.vocab, "width": c.width}
        if c.loop is not None:
            d["loop"] = {"start": c.loop.start, "stop": c.loop.stop, "times": c.loop.times}
        return d

    @staticmethod
    def _rotary(rot: Optional[Mapping[str, Any]]) -> Optional[Dict[str, Any]]:
        return None if rot is None else {"dims": rot["dims"], "theta": rot["base"]}

    @classmethod
    def _delta(cls, c: TirezenConfig, m: Mapping[str, Any], low_rank: bool, out_scale: float = 1.0) -> PartSpec:
        params = {"hidden_size": c.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
                  "conv": m["conv"], "eps": c.norm_eps, "out_scale": out_scale,
                  "decay": "channel" if low_rank else "head", "gate": "sigmoid_low_rank" if low_rank else "silu"}
        if low_rank:
            params.update(decay_rank=m["decay_rank"], gate_rank=m["gate_rank"])
        return PartSpec("gated_delta", params)

    @staticmethod
    def _delta_names(prefix: str, under: str, low_rank: bool) -> Dict[str, str]:
        names = {f"{prefix}q_proj": f"{under}q", f"{prefix}q_conv": f"{under}q.conv", f"{prefix}k_proj": f"{under}k",
                 f"{prefix}k_conv": f"{under}k.conv", f"{prefix}v_proj": f"{under}v", f"{prefix}v_conv": f"{under}v.conv",
                 f"{prefix}b_proj": f"{under}b", f"{prefix}A_log": f"{under}A_log", f"{prefix}norm": f"{under}norm",
                 f"{prefix}dt_bias": f"{under}dt_bias", f"{prefix}o_proj": f"{under}o"}
        if low_rank:
            names.update({f"{prefix}a1_proj": f"{under}a1", f"{prefix}a2_proj": f"{under}a2",
                          f"{prefix}g1_proj": f"{under}g1", f"{prefix}g2_proj": f"{under}g2"})
        else:
            names.update({f"{prefix}a_proj": f"{under}a", f"{prefix}g_proj": f"{under}g"})
        return names

    @classmethod
    def _layer(cls, c: TirezenConfig, i: int, layer: Mapping[str, Any]) -> LayerSpec:
        kind, m = layer["type"], layer["mixer"]
        names = {"norm_1.weight": "norm1"}
        if kind == "retention":
            mixer = PartSpec("retention", {"hidden_size": c.width, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                                           "decay": tuple(m["decay"]), "rotary": cls._rotary(m["rot"]), "eps": c.norm_eps})
            names.update({f"mixer.{p}_proj": f"mix.{p}" for p in ("q", "k", "v", "g", "o")})
        elif kind == "delta":
            mixer = cls._delta(c, m, low_rank=False)
            names.update(cls._delta_names("mixer.", "mix.", low_rank=False))
        else:
            left = m["left"]
            attention = PartSpec("general_attention", {
                "hidden_size": c.width, "num_heads": left["heads"], "num_kv_heads": left["kv_heads"], "head_dim": left["dim"],
                "v_head_dim": left["vdim"], "bias": True, "qk_norm_eps": c.norm_eps, "rotary": cls._rotary(left["rot"]),
                "scale": left["scale"], "softcap": left["softcap"], "sink": True, "window": None,
                "out_scale": m["left_scale"]})
            mixer = PartSpec("sum_of_mixers", {"mixers": {"left": attention,
                                                          "right": cls._delta(c, m["right"], True, m["right_scale"])}})
            for p in ("q", "k", "v"):
                names[f"mixer.left.{p}_proj"] = f"mix.left.{p}"
                names[f"mixer.left.{p}_bias"] = f"mix.left.{p}.b"
            names.update({"mixer.left.q_norm": "mix.left.q.norm", "mixer.left.k_norm": "mix.left.k.norm",
                          "mixer.left.o_proj": "mix.left.o"})
            names.update(cls._delta_names("mixer.right.", "mix.right.", low_rank=True))
        parts = {"norm_1": PartSpec("rms_norm", {"size": c.width, "eps": c.norm_eps, "one_plus": True}), "mixer": mixer}
        if layer["mlp"] is not None:
            parts["feed_forward"] = PartSpec("dense", {"hidden_size": c.width, "intermediate_size": layer["mlp"]["ff"],
                                                       "activation": "gelu_erf"})
            names.update({"feed_forward.up_proj": "mlp.up", "feed_forward.down_proj": "mlp.down"})
        return LayerSpec(block=PartSpec("parallel_residual"), parts=parts, weight_prefix=f"l{i}.", weight_names=names)

    @classmethod
    def model_spec(cls, c: TirezenConfig) -> ModelSpec:
        n = len(c.layers)
        if c.loop is None:
            schedule = [ScheduleEntry(i) for i in range(n)]
            extra = {}
        else:
            a, b, times = c.loop.start, c.loop.stop, c.loop.times
            schedule = [ScheduleEntry(i) for i in range(a)]
            for t in range(times):
                for i in range(a, b):
                    before = StreamInjection(embedding=t > 0, vector="loop_step", row=t) if i == a else None
                    schedule.append(ScheduleEntry(i, before=before))
            schedule += [ScheduleEntry(i) for i in range(b, n)]
            extra = {"loop_step": ("loop.step", (times, c.width))}
        return ModelSpec(
            architecture=ARCHITECTURE_NAME, hidden_size=c.width, vocab_size=c.vocab, max_position=MAX_POSITION,
            layers=tuple(cls._layer(c, i, layer) for i, layer in enumerate(c.layers)), schedule=tuple(schedule),
            final_norm=PartSpec("rms_norm", {"size": c.width, "eps": c.norm_eps, "one_plus": True}),
            embedding_name="embed", head_name="head", final_norm_names={"weight": "final.norm"}, extra_tensors=extra)


register_architecture(ARCHITECTURE_NAME, TirezenArchitecture, replace=True)
