"""Host-side mirror of the reference model loaders (metadata -> Configuration, tensor names ->
weight slots).  Mirrors ``model/loader/ModelLoader.java:47-108`` (type detection on
``general.name``), ``LlamaModelLoader.java:47-63`` / ``Qwen3ModelLoader.java:48-74``
(configuration keys), ``AbstractModelLoader.java:40-50`` (file_type -> quantisation) and
``AbstractModelLoader.java:186-195`` (tied output falls back to ``token_embd.weight``).
Weights stay in GGUF block layout; the native library repacks at upload.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

import json
import os
from dataclasses import field

from .gguf import GGMLType, GGUFFile
from .safetensors import SafetensorsFile

ARCH_LLAMA = 0
ARCH_QWEN3 = 1
ARCH_PHI3 = 2
ARCH_PIBIDRA = 3
ARCH_LATUSUN = 4
ARCH_LEROSUN = 5
ARCH_DINUZEN = 6

GGML_BF16 = 30  # ggml's id for bfloat16; layered plans take their safetensors tensors under it
_SAFETENSORS_TYPES = {"BF16": GGML_BF16, "F16": GGMLType.F16, "F32": GGMLType.F32}


@dataclass
class Configuration:
    arch: int
    quantization: str  # "FP16" | "Q8_0"
    dim: int
    hidden_dim: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    head_size: int
    vocab_size: int
    context_length: int
    rms_norm_eps: float
    rope_theta: float

    @property
    def q_dim(self):
        return self.n_heads * self.head_size

    @property
    def kv_dim(self):
        return self.n_kv_heads * self.head_size


@dataclass
class LayerSpec:
    """One layer of a layered model (``b200_layer_spec``): a mixer (windowed attention with its own key/value rows, or latent
    attention over a cached low-rank latent) and an optional feed-forward (dense gated, or a mixture of experts)."""
    heads: int
    kv_heads: int
    key_dim: int
    value_dim: int
    window: int
    bias_rows: int      # rows of the learned distance table (0: none)
    bias_far: float     # largest distance the logarithmic rows resolve
    score_scale: float
    softcap: float
    sink: bool = True
    gate: bool = True
    qkv_bias: bool = True
    qk_norm: bool = True
    ff_dim: int = 0     # 0: no feed-forward
    ff_act: str = "gelu_tanh"
    mixer: str = "window_attention"
    ff_kind: str = "dense"      # "dense" | "moe" (ff_dim = width of one expert)
    ff_experts: int = 0
    ff_top: int = 0
    # latent attention: key_dim = unrotated query/key size per head, rot_dim = rotated size (= size of the shared key part)
    rot_dim: int = 0
    kv_rank: int = 0
    kv_from: int = -1           # >= 0: reads that layer's cache and has no down-projection of its own
    rope_dims: int = 0          # leading entries of the rotated part that turn
    rope_layout: str = "half"   # "half": pair (i, i + dims/2) | "interleaved": pair (2i, 2i + 1)
    rope_base: float = 10000.0
    yarn: tuple = (0.0, 0.0, 0.0, 0.0)  # (factor, original length, fast, slow); factor 0: plain frequencies
    # windowed attention, each switchable on its own (rope_dims > 0 additionally rotates the leading entries of every query / key head)
    sink_learned: bool = False  # the sink's logit is a learned number per head instead of zero
    gate_per_head: bool = False  # one sigmoid gate per head instead of one per output entry
    value_from_key: bool = False  # no value projection: the values are the unrotated keys
    head_temp: bool = False     # a learned factor per head on the scores
    head_mix: bool = False      # scores mixed over the query heads before the softmax
    # gated delta rule: heads = value heads, kv_heads = query / key heads
    conv_taps: int = 0
    # differential attention (two score maps per head over the same values) and a per-slice q/k norm with one weight of size key_dim
    score_maps: int = 1
    diff_init: float = 0.0
    qk_head_norm: bool = False
    # "rglru": heads = diagonal blocks of the gates, value_dim = channels per block; "ssd": heads x value_dim values, key_dim = state
    # size, kv_heads = groups of B and C; mixer_norm_groups = parts of the read-out norm
    mixer_norm_groups: int = 1
    # mixture of experts
    moe_router: str = "sigmoid_input"   # | "softmax_output": softmax scores, selection by score + correction, weights on the outputs
    moe_identity: int = 0               # identity experts behind the real ones
    moe_scale: float = 1.0
    moe_shared_ff: int = 0              # width of the shared expert (0: none)


@dataclass
class LayeredConfiguration:
    """Configuration of a model given as a list of layers (``b200_layered_config``)."""
    arch: int
    width: int
    vocab_size: int
    context_length: int
    norm_eps: float
    embedding_scale: float
    layers: list = field(default_factory=list)
    loop: tuple | None = None  # (start, stop, times): layers [start, stop) run `times` passes over the same weights
    quantization: str = "BF16"
    # "sandwich": x += N(mixer(N x)); x += N(ff(N x)) | "parallel": x += mult * (mixer(LN1 x) + ff(LN2 x)) |
    # "prenorm": x += s1 * mixer(R x); x += s2 * ff(R x), R an RMS norm with one number as weight
    block: str = "sandwich"
    residual_mult: float = 1.0
    logit_softcap: float = 0.0
    # "outnorm": x += s1 * GN(mixer(shift x)); x += s2 * GN(ff(x)), GN = RMS norm in norm_groups parts on the sublayer's output
    norm_groups: int = 1
    token_shift: bool = False
    depth_average: bool = False

    @property
    def n_layers(self):
        return len(self.layers)

    @property
    def dim(self):
        return self.width

    def layer_runs(self) -> int:
        if self.loop is None or self.loop[1] <= self.loop[0]:
            return len(self.layers)
        return len(self.layers) + (self.loop[2] - 1) * (self.loop[1] - self.loop[0])


class UnsupportedModel(Exception):
    """Maps to the reference's UnsupportedOperationException (ForwardPlanFactory.java:84-87)."""


def detect_model_type(metadata: dict) -> str:
    name = metadata.get("general.name")
    if name is not None:
        low = name.lower()
        for key, typ in (("granite", "GRANITE"), ("devstral", "DEVSTRAL_2"), ("mistral", "MISTRAL"),
                         ("llama", "LLAMA_3"), ("qwen2", "QWEN_2"), ("qwen3", "QWEN_3"),
                         ("deepseek r1 distill", "DEEPSEEK_R1_DISTILL_QWEN"), ("phi3", "PHI_3"), ("phi-3", "PHI_3")):
            if key in low:
                return typ
    return "UNKNOWN"


def _quantization(metadata: dict) -> str:
    ft = int(metadata["general.file_type"])
    if ft == 1:
        return "FP16"
    if ft == 7:
        return "Q8_0"
    if ft in (14, 15, 16, 17, 18):  # Q4_K_S/M, Q5_K_S/M, Q6_K: the accelerator path computes in Q8_0 (AbstractModelLoader.java:45-47)
        return "Q8_0"
    raise UnsupportedModel(f"Unsupported quantization format: {ft} (as int).")


class Model:
    """Configuration + raw tensor views.  ``tensors[name] = (ggml_type, dims, uint8 ndarray)``."""

    def __init__(self, gguf: GGUFFile | None, config: Configuration, model_type: str, tensors: dict | None = None):
        self.gguf = gguf
        self.configuration = config
        self.model_type = model_type
        self.tensors = dict(tensors) if tensors is not None else {}
        if gguf is not None:
            for name, ti in gguf.tensor_infos.items():
                if name == "rope_freqs.weight":  # GGUF.java:121-124
                    continue
                self.tensors[name] = (ti.ggml_type, ti.dims, gguf.tensor_bytes(name))
        self.plan = None  # Model.setTornadoVMPlan
        self.latest_token = None


def model_from_tensors(shape, quant: int, tensors: dict, context_length: int) -> Model:
    """In-memory model (bench: synthetic weights never touch the disk)."""
    arch = {"llama": ARCH_LLAMA, "qwen3": ARCH_QWEN3, "phi3": ARCH_PHI3}[shape.arch]
    cfg = Configuration(arch, "Q8_0" if quant == GGMLType.Q8_0 else "FP16",
                        shape.dim, shape.hidden, shape.n_layers, shape.n_heads, shape.n_kv_heads, shape.head_size,
                        shape.vocab, context_length, float(shape.eps), float(shape.rope_theta))
    return Model(None, cfg, {"llama": "LLAMA_3", "qwen3": "QWEN_3", "phi3": "PHI_3"}[shape.arch], tensors)


def pibidra_configuration(cfg: dict, tensor_shapes: dict, context_length: int) -> LayeredConfiguration:
    """config.json of a Pibidra model -> LayeredConfiguration.  Every size comes from the file; the shape of each layer's
    distance table gives its row count."""
    layers = []
    for i, lc in enumerate(cfg["layers"]):
        if lc["type"] != "attention":
            raise UnsupportedModel(f"layer {i}: mixer type {lc['type']!r} (Pibidra layers are 'attention')")
        m, mlp = lc["mixer"], lc.get("mlp")
        if mlp is not None and mlp.get("kind") != "dense":
            raise UnsupportedModel(f"layer {i}: feed-forward kind {mlp.get('kind')!r}")
        rel = tensor_shapes.get(f"l{i}.mix.rel")
        if rel is None or len(rel) != 2 or rel[1] != int(m["heads"]):
            raise UnsupportedModel(f"layer {i}: distance table l{i}.mix.rel missing or not [rows][heads]")
        layers.append(LayerSpec(
            heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), key_dim=int(m["dim"]), value_dim=int(m["vdim"]),
            window=int(m["mask"]["size"]), bias_rows=int(rel[0]), bias_far=float(m["bias_max"]), score_scale=float(m["scale"]),
            softcap=float(m["softcap"]), ff_dim=int(mlp["ff"]) if mlp is not None else 0))
    loop = cfg.get("loop")
    return LayeredConfiguration(
        ARCH_PIBIDRA, int(cfg["width"]), int(cfg["vocab"]), int(context_length), float(cfg["norm"]["eps"]), float(cfg["embedding"]["scale"]),
        layers, (int(loop["start"]), int(loop["stop"]), int(loop["times"])) if loop else None)


# Latusun: mixer type -> (pairing of the rotation, output gate)
LATUSUN_MIXERS = {"latent_attention": ("half", True), "latent_attention_2": ("interleaved", False)}


def latusun_configuration(cfg: dict, tensor_shapes: dict, context_length: int) -> LayeredConfiguration:
    """config.json of a Latusun model -> LayeredConfiguration: parallel blocks of latent attention and a sigmoid-routed mixture of
    SiLU experts.  Every size and every constant that can differ between models comes from the file."""
    layers = []
    for i, lc in enumerate(cfg["layers"]):
        if lc["type"] not in LATUSUN_MIXERS:
            raise UnsupportedModel(f"layer {i}: mixer type {lc['type']!r} (Latusun layers are {sorted(LATUSUN_MIXERS)})")
        layout, gate = LATUSUN_MIXERS[lc["type"]]
        m, mlp = lc["mixer"], lc.get("mlp")
        if mlp is not None and mlp.get("kind") != "moe":
            raise UnsupportedModel(f"layer {i}: feed-forward kind {mlp.get('kind')!r}")
        rot = m["rot"]
        sc = rot.get("scaling")
        kv_from = m.get("kv_from")
        if f"l{i}.mix.dkv" in tensor_shapes and kv_from is not None:
            raise UnsupportedModel(f"layer {i}: reads layer {kv_from}'s cache but carries a down-projection of its own")
        layers.append(LayerSpec(
            heads=int(m["heads"]), kv_heads=1, key_dim=int(m["dim"]), value_dim=int(m["vdim"]), window=int(context_length), bias_rows=0, bias_far=0.0,
            score_scale=float(m["scale"]), softcap=0.0, sink=False, gate=gate, qkv_bias=False, qk_norm=False,
            ff_dim=int(mlp["expert"]["ff"]) if mlp is not None else 0, ff_act="silu", mixer="latent_attention",
            ff_kind="moe" if mlp is not None else "dense", ff_experts=int(mlp["router"]["experts"]) if mlp is not None else 0,
            ff_top=int(mlp["router"]["top"]) if mlp is not None else 0,
            rot_dim=int(m["rot_dim"]), kv_rank=int(m["kv_rank"]), kv_from=-1 if kv_from is None else int(kv_from),
            rope_dims=int(rot["dims"]), rope_layout=layout, rope_base=float(rot["base"]),
            yarn=(float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"])) if sc else (0.0, 0.0, 0.0, 0.0)))
    return LayeredConfiguration(
        ARCH_LATUSUN, int(cfg["width"]), int(cfg["vocab"]), int(context_length), float(cfg["norm"]["eps"]), 1.0, layers, None,
        block="parallel", residual_mult=float(cfg.get("residual_mult", 1.0)), logit_softcap=float(cfg.get("logit_softcap") or 0.0))


def lerosun_configuration(cfg: dict, tensor_shapes: dict, context_length: int) -> LayeredConfiguration:
    """config.json of a Lerosun model -> LayeredConfiguration: pre-norm blocks whose mixer is a sliding-window attention (partial
    rotation, values = unrotated keys, per-head temperature, head-mixed scores, learned sink, per-head gate) or a gated delta rule,
    and a gated ReLU feed-forward.  Every size and every constant that can differ between models comes from the file."""
    layers = []
    for i, lc in enumerate(cfg["layers"]):
        m, mlp = lc["mixer"], lc.get("mlp")
        if mlp is not None and mlp.get("kind") != "dense":
            raise UnsupportedModel(f"layer {i}: feed-forward kind {mlp.get('kind')!r}")
        ff = dict(ff_dim=int(mlp["ff"]) if mlp is not None else 0, ff_act="relu")
        if lc["type"] == "attention":
            rot = m.get("rot")
            layers.append(LayerSpec(
                heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), key_dim=int(m["dim"]), value_dim=int(m["vdim"]), window=int(m["mask"]["size"]),
                bias_rows=0, bias_far=0.0, score_scale=float(m["scale"]), softcap=0.0, sink=True, gate=True, qkv_bias=True, qk_norm=False,
                rope_dims=int(rot["dims"]) if rot else 0, rope_layout="half", rope_base=float(rot["base"]) if rot else 10000.0,
                sink_learned=True, gate_per_head=True, value_from_key=True, head_temp=True, head_mix=True, **ff))
        elif lc["type"] == "delta":
            layers.append(LayerSpec(
                heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), key_dim=int(m["dim"]), value_dim=int(m["vdim"]), window=1, bias_rows=0, bias_far=0.0,
                score_scale=1.0, softcap=0.0, sink=False, gate=True, qkv_bias=False, qk_norm=False, mixer="gated_delta", conv_taps=int(m["conv"]), **ff))
        else:
            raise UnsupportedModel(f"layer {i}: mixer type {lc['type']!r} (Lerosun layers are 'attention' or 'delta')")
    loop = cfg.get("loop")
    return LayeredConfiguration(
        ARCH_LEROSUN, int(cfg["width"]), int(cfg["vocab"]), int(context_length), float(cfg["norm"]["eps"]), 1.0, layers,
        (int(loop["start"]), int(loop["stop"]), int(loop["times"])) if loop else None, block="prenorm")


def dinuzen_configuration(cfg: dict, tensor_shapes: dict, context_length: int) -> LayeredConfiguration:
    """config.json of a Dinuzen model -> LayeredConfiguration: blocks with the norm on the sublayer's output, token shift and depth
    average; per layer a real-gated linear recurrent unit, a state-space recurrence or a differential attention, and a plain GELU
    feed-forward or a softmax-routed mixture of experts.  All sizes and all model-dependent constants are read from
    the file."""
    layers = []
    for i, lc in enumerate(cfg["layers"]):
        m, mlp = lc["mixer"], lc.get("mlp")
        if mlp is None:
            ff = dict(ff_dim=0)
        elif mlp.get("kind") == "dense":
            ff = dict(ff_dim=int(mlp["ff"]), ff_act="gelu_erf", ff_kind="dense_plain")
        elif mlp.get("kind") == "moe":
            r, sh = mlp["router"], mlp.get("shared")
            ff = dict(ff_dim=int(mlp["expert"]["ff"]), ff_act="silu", ff_kind="moe", ff_experts=int(r["experts"]), ff_top=int(r["top"]),
                      moe_router="softmax_output", moe_identity=int(r.get("identity", 0)), moe_scale=float(r.get("scale", 1.0)),
                      moe_shared_ff=int(sh["ff"]) if sh else 0)
        else:
            raise UnsupportedModel(f"layer {i}: feed-forward kind {mlp.get('kind')!r}")
        base = dict(bias_rows=0, bias_far=0.0, sink=False, gate=False, qkv_bias=False, qk_norm=False)
        if lc["type"] == "attention":
            rot = m["rot"]
            sc = rot.get("scaling")
            kv_from = m.get("kv_from")
            if kv_from is not None and f"l{i}.mix.k" in tensor_shapes:
                raise UnsupportedModel(f"layer {i}: reads layer {kv_from}'s keys and values but carries projections of its own")
            layers.append(LayerSpec(
                heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), key_dim=int(m["dim"]), value_dim=int(m["vdim"]), window=int(context_length),
                score_scale=float(m["scale"]), softcap=float(m.get("softcap") or 0.0), score_maps=2, diff_init=float(m["diff"]), qk_head_norm=True,
                kv_from=-1 if kv_from is None else int(kv_from), rope_dims=int(rot["dims"]), rope_layout="interleaved", rope_base=float(rot["base"]),
                yarn=(float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"])) if sc else (0.0, 0.0, 0.0, 0.0), **base, **ff))
        elif lc["type"] == "rglru":
            blocks, width = int(m["blocks"]), int(m["width"])
            if blocks <= 0 or width % blocks:
                raise UnsupportedModel(f"layer {i}: {width} channels in {blocks} blocks")
            layers.append(LayerSpec(heads=blocks, kv_heads=blocks, key_dim=width // blocks, value_dim=width // blocks, window=1, score_scale=1.0, softcap=0.0,
                                    mixer="rglru", conv_taps=int(m["conv"]), **base, **ff))
        elif lc["type"] == "mamba2":
            layers.append(LayerSpec(heads=int(m["heads"]), kv_heads=int(m["groups"]), key_dim=int(m["state"]), value_dim=int(m["vdim"]), window=1, score_scale=1.0,
                                    softcap=0.0, mixer="ssd", conv_taps=int(m["conv"]), mixer_norm_groups=int(m.get("norm_groups", 1)), **base, **ff))
        else:
            raise UnsupportedModel(f"layer {i}: mixer type {lc['type']!r} (Dinuzen layers are 'attention', 'rglru' or 'mamba2')")
    return LayeredConfiguration(
        ARCH_DINUZEN, int(cfg["width"]), int(cfg["vocab"]), int(context_length), float(cfg["norm"]["eps"]), 1.0, layers, None,
        block="outnorm", norm_groups=int(cfg["norm"].get("groups", 1)), token_shift=True, depth_average=True)


# config.json "architecture" -> (model type, configuration builder): the registry of safetensors model directories
CONFIG_ARCHITECTURES = {"Pibidra": ("PIBIDRA", pibidra_configuration), "Latusun": ("LATUSUN", latusun_configuration),
                        "Lerosun": ("LEROSUN", lerosun_configuration), "Dinuzen": ("DINUZEN", dinuzen_configuration)}
DEFAULT_LAYERED_CONTEXT = 4096


def load_model_dir(path: str, context_length: int = -1) -> Model:
    """A directory with config.json + model.safetensors; the model class is chosen by config.json's "architecture"."""
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    arch = cfg.get("architecture")
    if arch not in CONFIG_ARCHITECTURES:
        raise UnsupportedModel(f"architecture {arch!r} is not one of {sorted(CONFIG_ARCHITECTURES)}")
    typ, make = CONFIG_ARCHITECTURES[arch]
    st = SafetensorsFile(os.path.join(path, "model.safetensors"))
    tensors, shapes = {}, {}
    for name, (dt, shape, _, _) in st.infos.items():
        if dt not in _SAFETENSORS_TYPES:
            raise UnsupportedModel(f"tensor {name}: dtype {dt}")
        shapes[name] = shape
        tensors[name] = (_SAFETENSORS_TYPES[dt], tuple(reversed(shape)), st.tensor_bytes(name))  # dims[0] = innermost, as in GGUF
    config = make(cfg, shapes, DEFAULT_LAYERED_CONTEXT if context_length < 0 else context_length)
    m = Model(None, config, typ, tensors)
    m.safetensors = st
    return m


def load_model(path: str, context_length: int = -1) -> Model:
    """``ModelLoader.loadModel(Path,int,boolean,boolean)`` (ModelLoader.java:113-120); a directory is a safetensors model."""
    if os.path.isdir(path):
        return load_model_dir(path, context_length)
    g = GGUFFile(path)
    md = g.metadata
    typ = detect_model_type(md)
    q = _quantization(md)
    if typ == "LLAMA_3" or typ == "MISTRAL":
        # Mistral runs the same forward as Llama (Mistral.java -> InferenceCore.forwardJava; weights in the same
        # LlamaStandardWeights slots, MistralModelLoader.java:92-113).  Differences are host-side only: the context is
        # clamped to the model's (MistralModelLoader.java:45-46) and the vocabulary size may come from the token list.
        vocab = md.get("llama.vocab_size")
        if vocab is None:
            vocab = len(md["tokenizer.ggml.tokens"])
        model_ctx = int(md["llama.context_length"])
        n_heads = int(md["llama.attention.head_count"])
        dim = int(md["llama.embedding_length"])
        if typ == "MISTRAL":
            ctx = model_ctx if (context_length < 0 or model_ctx < context_length) else context_length
        else:  # withContextLength(contextLength): LlamaConfiguration keeps the requested length when >= 0
            ctx = model_ctx if context_length < 0 else context_length
        cfg = Configuration(
            ARCH_LLAMA, q, dim, int(md["llama.feed_forward_length"]), int(md["llama.block_count"]), n_heads,
            int(md.get("llama.attention.head_count_kv", n_heads)), dim // n_heads, int(vocab), ctx,
            float(md.get("llama.attention.layer_norm_rms_epsilon", 1e-5)), float(md.get("llama.rope.freq_base", 10000.0)))
    elif typ == "QWEN_3":
        model_ctx = int(md["qwen3.context_length"])
        ctx = model_ctx if (context_length < 0 or model_ctx < context_length) else context_length
        vocab = md.get("qwen3.vocab_size")
        if vocab is None:
            vocab = len(md["tokenizer.ggml.tokens"])
        n_heads = int(md["qwen3.attention.head_count"])
        if int(md["qwen3.attention.key_length"]) != int(md["qwen3.attention.value_length"]):
            raise UnsupportedModel("key_length != value_length")
        cfg = Configuration(
            ARCH_QWEN3, q, int(md["qwen3.embedding_length"]), int(md["qwen3.feed_forward_length"]),
            int(md["qwen3.block_count"]), n_heads, int(md.get("qwen3.attention.head_count_kv", n_heads)),
            int(md["qwen3.attention.key_length"]), int(vocab), ctx,
            float(md["qwen3.attention.layer_norm_rms_epsilon"]), float(md["qwen3.rope.freq_base"]))
    elif typ == "PHI_3":
        # Phi3ModelLoader.createConfiguration (Phi3ModelLoader.java:51-71): head size = dim / heads, the context is the requested one
        # (the RoPE table is precomputed for the model's), the vocabulary size is the token list's.
        n_heads = int(md["phi3.attention.head_count"])
        dim = int(md["phi3.embedding_length"])
        model_ctx = int(md["phi3.context_length"])
        vocab = len(md["tokenizer.ggml.tokens"]) if "tokenizer.ggml.tokens" in md else int(md["phi3.vocab_size"])
        cfg = Configuration(
            ARCH_PHI3, q, dim, int(md["phi3.feed_forward_length"]), int(md["phi3.block_count"]), n_heads,
            int(md.get("phi3.attention.head_count_kv", n_heads)), dim // n_heads, int(vocab), model_ctx if context_length < 0 else context_length,
            float(md.get("phi3.attention.layer_norm_rms_epsilon", 1e-5)), float(md.get("phi3.rope.freq_base", 10000.0)))
    else:
        raise UnsupportedModel(f"model type {typ} is outside the B200 hot-path scope (Llama / Mistral / Qwen3 / Phi-3 forward passes only)")
    return Model(g, cfg, typ)


def tensor_as_f32(model: Model, name: str) -> np.ndarray:
    """Dequantise a whole tensor the way ``FloatTensor.getFloat`` does (tests / debugging)."""
    tt, dims, raw = model.tensors[name]
    if tt == GGMLType.F32:
        return raw.view("<f4").copy()
    if tt == GGMLType.F16:
        return raw.view("<f2").astype(np.float32)
    blocks = raw.reshape(-1, 34)
    d = blocks[:, :2].copy().view("<f2").astype(np.float32)
    q = blocks[:, 2:].view(np.int8).astype(np.float32)
    return (q * d).reshape(-1)
