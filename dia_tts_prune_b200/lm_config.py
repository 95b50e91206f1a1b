"""Configuration schemas of the decoder-only language models (``config.json`` of a model folder): Pubopel, Kupelix,
Luketar and Fipadra.

Every size and every per-model constant comes from the file.  Optional entries that are absent switch their
mechanism off: no ``mask`` is full causal attention, no ``softcap`` leaves scores uncapped, ``mlp: null`` is a layer
without feed-forward, no ``shared`` a mixture without shared expert.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Annotated, Literal, Optional, Union

from pydantic import BaseModel, Field


class MaskConfig(BaseModel, frozen=True):
    size: int = Field(gt=0)                      # key j is seen from i when i - j < size ...
    keep_first: int = Field(default=0, ge=0)     # ... or j < keep_first


class AttentionMixerConfig(BaseModel, frozen=True):
    heads: int = Field(gt=0)
    kv_heads: int = Field(gt=0)
    dim: int = Field(gt=0)
    vdim: int = Field(gt=0)
    scale: float
    softcap: Optional[float] = None
    mask: Optional[MaskConfig] = None


class ExpertConfig(BaseModel, frozen=True):
    ff: int = Field(gt=0)


class RouterConfig(BaseModel, frozen=True):
    experts: int = Field(gt=0)
    top: int = Field(gt=0)


class MlpConfig(BaseModel, frozen=True):
    kind: Literal["moe"] = "moe"
    expert: ExpertConfig
    router: RouterConfig
    shared: Optional[ExpertConfig] = None


class LayerConfig(BaseModel, frozen=True):
    type: Literal["attention"]
    mixer: AttentionMixerConfig
    mlp: Optional[MlpConfig] = None


class TapConfig(BaseModel, frozen=True):
    taps: int = Field(ge=1)


class NormConfig(BaseModel, frozen=True):
    eps: float = Field(ge=0.0)


class PubopelConfig(BaseModel, frozen=True):
    architecture: Literal["Pubopel"] = "Pubopel"
    vocab: int = Field(gt=0)
    width: int = Field(gt=0)
    layers: list[LayerConfig] = Field(min_length=1)
    canon: TapConfig
    norm: NormConfig

    @classmethod
    def load(cls, path: str | Path) -> "PubopelConfig":
        return cls.model_validate(json.loads(Path(path).read_text(encoding="utf-8")))

    def check(self) -> None:
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if m.heads % m.kv_heads:
                raise ValueError(f"layer {i}: heads ({m.heads}) must be a multiple of kv_heads ({m.kv_heads})")
            if m.vdim != m.dim:
                raise ValueError(f"layer {i}: the values are the projected keys, so vdim ({m.vdim}) must equal dim ({m.dim})")
            if layer.mlp is not None and layer.mlp.router.top > layer.mlp.router.experts:
                raise ValueError(f"layer {i}: top ({layer.mlp.router.top}) exceeds experts ({layer.mlp.router.experts})")


# ---- Kupelix: parallel layers (one layer norm feeds mixer and feed-forward), three mixers, an optional repeated block ----
class RotScalingConfig(BaseModel, frozen=True):
    factor: float = Field(gt=0.0)
    low: float
    high: float
    original: float = Field(gt=0.0)


class RotConfig(BaseModel, frozen=True):
    base: float = Field(gt=0.0)
    dims: int = Field(ge=0)                      # leading channels of every head that turn with the position
    scaling: Optional[RotScalingConfig] = None


class TalkAttentionMixerConfig(BaseModel, frozen=True):
    heads: int = Field(gt=0)
    kv_heads: Optional[int] = Field(default=None, gt=0)
    dim: int = Field(gt=0)
    vdim: int = Field(gt=0)
    scale: float
    rot: Optional[RotConfig] = None


class Hgrn2MixerConfig(BaseModel, frozen=True):
    heads: int = Field(gt=0)
    dim: int = Field(gt=0)
    vdim: int = Field(gt=0)


class ChannelDeltaMixerConfig(BaseModel, frozen=True):
    heads: int = Field(gt=0)
    kv_heads: Optional[int] = Field(default=None, gt=0)
    dim: int = Field(gt=0)
    vdim: int = Field(gt=0)
    conv: int = Field(ge=1)                      # taps of the short convolutions of q, k, v


class DenseMlpConfig(BaseModel, frozen=True):
    kind: Literal["dense"] = "dense"
    ff: int = Field(gt=0)


class KupelixAttentionLayer(BaseModel, frozen=True):
    type: Literal["attention"]
    mixer: TalkAttentionMixerConfig
    mlp: Optional[DenseMlpConfig] = None


class KupelixHgrn2Layer(BaseModel, frozen=True):
    type: Literal["hgrn2"]
    mixer: Hgrn2MixerConfig
    mlp: Optional[DenseMlpConfig] = None


class KupelixDeltaLayer(BaseModel, frozen=True):
    type: Literal["channel_delta"]
    mixer: ChannelDeltaMixerConfig
    mlp: Optional[DenseMlpConfig] = None


KupelixLayer = Annotated[Union[KupelixAttentionLayer, KupelixHgrn2Layer, KupelixDeltaLayer], Field(discriminator="type")]


class LoopConfig(BaseModel, frozen=True):
    start: int = Field(ge=0)                     # layers start .. stop-1 run `times` times in a row with the same weights
    stop: int = Field(ge=0)
    times: int = Field(ge=1)


class KupelixConfig(BaseModel, frozen=True):
    architecture: Literal["Kupelix"] = "Kupelix"
    vocab: int = Field(gt=0)
    width: int = Field(gt=0)
    layers: list[KupelixLayer] = Field(min_length=1)
    loop: Optional[LoopConfig] = None
    norm: NormConfig
    logit_scale: float = 1.0

    @classmethod
    def load(cls, path: str | Path) -> "KupelixConfig":
        return cls.model_validate(json.loads(Path(path).read_text(encoding="utf-8")))

    def check(self) -> None:
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            g = getattr(m, "kv_heads", None) or m.heads
            if m.heads % g:
                raise ValueError(f"layer {i}: heads ({m.heads}) must be a multiple of kv_heads ({g})")
            rot = getattr(m, "rot", None)
            if rot is not None and (rot.dims % 2 or rot.dims > m.dim):
                raise ValueError(f"layer {i}: rot.dims ({rot.dims}) must be even and at most dim ({m.dim})")
        if self.loop is not None and not (0 <= self.loop.start < self.loop.stop <= len(self.layers)):
            raise ValueError("loop: start < stop <= number of layers is required")

    def runs(self) -> list[tuple[int, bool]]:
        """(layer index, whether a pass of the repeated block starts here) in execution order."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        a, b = self.loop.start, self.loop.stop
        out = [(i, False) for i in range(a)]
        for _ in range(self.loop.times):
            out += [(i, i == a) for i in range(a, b)]
        return out + [(i, False) for i in range(b, n)]


# ---- Luketar: pre-norm sublayers over hyper-connected residual streams, latent attention / mLSTM mixers, clamped gated units ----
class LatentAttentionMixerConfig(BaseModel, frozen=True):
    heads: int = Field(gt=0)
    dim: int = Field(gt=0)                       # query / key size per head
    vdim: int = Field(gt=0)
    q_rank: int = Field(gt=0)                    # size of the query latent
    kv_rank: int = Field(gt=0)                   # size of the cached key/value latent
    scale: float


class MlstmMixerConfig(BaseModel, frozen=True):
    heads: int = Field(gt=0)
    dim: int = Field(gt=0)
    vdim: int = Field(gt=0)
    gate_cap: float = Field(gt=0.0)              # gate pre-activations z become cap tanh(z / cap)


class GatedUnitConfig(BaseModel, frozen=True):
    ff: int = Field(gt=0)
    limit: float = Field(gt=0.0)                 # clamp of the gate (from above) and of the up branch (both sides)


class GatedDenseMlpConfig(BaseModel, frozen=True):
    kind: Literal["dense"]
    ff: int = Field(gt=0)
    limit: float = Field(gt=0.0)


class GatedMoeMlpConfig(BaseModel, frozen=True):
    kind: Literal["moe"]
    expert: GatedUnitConfig
    router: RouterConfig
    shared: Optional[GatedUnitConfig] = None


GatedMlp = Annotated[Union[GatedDenseMlpConfig, GatedMoeMlpConfig], Field(discriminator="kind")]


class LuketarAttentionLayer(BaseModel, frozen=True):
    type: Literal["latent_attention"]
    mixer: LatentAttentionMixerConfig
    mlp: Optional[GatedMlp] = None
    weights_of: Optional[int] = Field(default=None, ge=0)   # this layer runs with that layer's weights and a state of its own


class LuketarMlstmLayer(BaseModel, frozen=True):
    type: Literal["mlstm"]
    mixer: MlstmMixerConfig
    mlp: Optional[GatedMlp] = None
    weights_of: Optional[int] = Field(default=None, ge=0)


LuketarLayer = Annotated[Union[LuketarAttentionLayer, LuketarMlstmLayer], Field(discriminator="type")]


class EmbeddingConfig(BaseModel, frozen=True):
    scale: float = 1.0


class LuketarConfig(BaseModel, frozen=True):
    architecture: Literal["Luketar"] = "Luketar"
    vocab: int = Field(gt=0)
    width: int = Field(gt=0)
    layers: list[LuketarLayer] = Field(min_length=1)
    norm: NormConfig
    embedding: EmbeddingConfig = EmbeddingConfig()
    streams: Optional[int] = Field(default=None, ge=1, le=8)    # residual streams with hyper-connections; None: one plain residual

    @classmethod
    def load(cls, path: str | Path) -> "LuketarConfig":
        return cls.model_validate(json.loads(Path(path).read_text(encoding="utf-8")))

    def weight_layer(self, i: int) -> int:
        """The layer whose tensors layer ``i`` uses (a named layer that itself names another one is followed)."""
        seen = {i}
        while self.layers[i].weights_of is not None:
            i = self.layers[i].weights_of
            if i in seen or i >= len(self.layers):
                raise ValueError("weights_of must lead to a layer that has weights of its own")
            seen.add(i)
        return i

    def check(self) -> None:
        for i, layer in enumerate(self.layers):
            j = self.weight_layer(i)
            if j != i and self.layers[j].type != layer.type:     # (the sizes and constants that run are layer j's)
                raise ValueError(f"layer {i}: its type differs from layer {j}, whose weights it uses")
            f = layer.mlp
            if f is not None and f.kind == "moe" and f.router.top > f.router.experts:
                raise ValueError(f"layer {i}: top ({f.router.top}) exceeds experts ({f.router.experts})")


# ---- Fipadra: parallel layers with two RMS norms (x += mixer(norm1 x) + ff(norm2 x)); gated delta rule / latent attention with a
# ---- turned key part and a sliding window / retention; squared-relu dense units or a grouped, softmax-scored mixture ----
class GatedDeltaMixerConfig(BaseModel, frozen=True):
    heads: int = Field(gt=0)
    kv_heads: Optional[int] = Field(default=None, gt=0)
    dim: int = Field(gt=0)
    vdim: int = Field(gt=0)
    conv: int = Field(ge=1)                      # taps of the short convolutions of q, k, v


class WindowConfig(BaseModel, frozen=True):
    size: int = Field(gt=0)                      # position i sees j when 0 <= i - j < size


class RotaryLatentMixerConfig(BaseModel, frozen=True):
    heads: int = Field(gt=0)
    dim: int = Field(gt=0)                       # query / key channels per head that do not turn
    rot_dim: int = Field(default=0, ge=0)        # ... and that turn with the position (the key's are shared by all heads)
    vdim: int = Field(gt=0)
    q_rank: int = Field(gt=0)
    kv_rank: int = Field(gt=0)
    scale: float
    rot: Optional[RotConfig] = None
    mask: Optional[WindowConfig] = None


class RetentionMixerConfig(BaseModel, frozen=True):
    heads: int = Field(gt=0)
    dim: int = Field(gt=0)
    vdim: int = Field(gt=0)
    decay: list[float]                           # one fixed decay per head
    rot: Optional[RotConfig] = None


class GroupConfig(BaseModel, frozen=True):
    count: int = Field(ge=1)                     # equal groups of neighbouring router outputs
    keep: int = Field(ge=1)                      # groups a token may choose from


class GroupedRouterConfig(BaseModel, frozen=True):
    experts: int = Field(gt=0)
    top: int = Field(gt=0)
    identity: int = Field(default=0, ge=0)       # router outputs behind the experts' whose expert returns its input
    scale: float = 1.0
    groups: Optional[GroupConfig] = None


class GroupedMoeMlpConfig(BaseModel, frozen=True):
    kind: Literal["moe"]
    expert: GatedUnitConfig
    router: GroupedRouterConfig
    shared: Optional[GatedUnitConfig] = None


FipadraMlp = Annotated[Union[DenseMlpConfig, GroupedMoeMlpConfig], Field(discriminator="kind")]


class FipadraDeltaLayer(BaseModel, frozen=True):
    type: Literal["delta"]
    mixer: GatedDeltaMixerConfig
    mlp: Optional[FipadraMlp] = None


class FipadraAttentionLayer(BaseModel, frozen=True):
    type: Literal["latent_attention"]
    mixer: RotaryLatentMixerConfig
    mlp: Optional[FipadraMlp] = None


class FipadraRetentionLayer(BaseModel, frozen=True):
    type: Literal["retention"]
    mixer: RetentionMixerConfig
    mlp: Optional[FipadraMlp] = None


FipadraLayer = Annotated[Union[FipadraDeltaLayer, FipadraAttentionLayer, FipadraRetentionLayer], Field(discriminator="type")]


class FipadraConfig(BaseModel, frozen=True):
    architecture: Literal["Fipadra"] = "Fipadra"
    vocab: int = Field(gt=0)
    width: int = Field(gt=0)
    layers: list[FipadraLayer] = Field(min_length=1)
    norm: NormConfig
    logit_scale: float = 1.0

    @classmethod
    def load(cls, path: str | Path) -> "FipadraConfig":
        return cls.model_validate(json.loads(Path(path).read_text(encoding="utf-8")))

    def check(self) -> None:
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            g = getattr(m, "kv_heads", None) or m.heads
            if m.heads % g:
                raise ValueError(f"layer {i}: heads ({m.heads}) must be a multiple of kv_heads ({g})")
            rot = getattr(m, "rot", None)
            if rot is not None:
                turning = m.rot_dim if layer.type == "latent_attention" else m.dim
                if rot.dims % 2 or rot.dims > turning:
                    raise ValueError(f"layer {i}: rot.dims ({rot.dims}) must be even and at most {turning}")
            if layer.type == "retention" and len(m.decay) != m.heads:
                raise ValueError(f"layer {i}: decay needs one number per head")
            f = layer.mlp
            if f is not None and f.kind == "moe":
                n = f.router.experts + f.router.identity
                per = n
                if f.router.groups is not None:
                    if n % f.router.groups.count or f.router.groups.keep > f.router.groups.count:
                        raise ValueError(f"layer {i}: {n} router outputs do not form {f.router.groups.count} equal groups")
                    per = f.router.groups.keep * (n // f.router.groups.count)
                if f.router.top > per:
                    raise ValueError(f"layer {i}: top ({f.router.top}) exceeds the router outputs a token may choose from ({per})")


CONFIGS = {"pubopel": PubopelConfig, "kupelix": KupelixConfig, "luketar": LuketarConfig, "fipadra": FipadraConfig}


def load_config(raw: dict):
    """The configuration object of a language model's ``config.json`` dictionary, by its ``architecture``."""
    name = str(raw.get("architecture", "")).lower()
    if name not in CONFIGS:
        raise NotImplementedError(f"no language-model configuration for architecture {raw.get('architecture')!r}")
    return CONFIGS[name].model_validate(raw)
