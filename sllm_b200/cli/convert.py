"""`sllm-convert-gguf`: writes a GGUF file plus its derived lock.

Kinds:
  random-llama   seeded random-init weights of a named shape (`--artifact llama3-8b`), for benchmarks and tests; the
                 mixture-of-experts (`moe-120b`, `qwen35-moe`, `tiny-moe`, `tiny-shared-moe`) and hybrid
                 (`qwen35-hybrid`, `qwen35-moe-hybrid`, `tiny-qwen35`, `tiny-qwen35-moe`) shapes are written through models/family_io.py with MXFP4 experts
  hf-llama       a Llama-style Hugging Face checkpoint (config.json + safetensors) from a directory that is first
                 verified against its model lock (`--lock lock.json --cache DIR`)
  mixed-precision  a compressed-tensors checkpoint with FP8 channel-scaled attention projections, NVFP4 MLP
                 projections and per-layer static FP8 KV scales (formats/quantized_model.py); same lock verification.
                 The file keeps the FP8 matrices block-scaled, the NVFP4 matrices as GGML type-40 blocks with their
                 outer scales, and the KV scales in the model configuration
  hf-qwen35      a Qwen3.5 checkpoint (gated-delta-net / full-attention hybrid; `qwen3_5_text` with a dense MLP or
                 `qwen3_5_moe_text` with routed MXFP4 experts stored as packed U8 values plus E8M0 `weight_scale`
                 planes and a gated shared expert); the decoder tensors under `model.language_model.` are consumed,
                 `model.visual.*` and `mtp.*` are recorded as known-unconsumed; same lock verification
`--weight-format bf16|fp8` selects the resident encoding (fp8 = E4M3FN with FP32 scales per 1x128 block).
`--dry-run` validates inputs and prints the plan without writing.  (Reference: crates/sllm-server/src/bin/
sllm-convert-gguf.rs flags --kind --lock --cache --artifact --manifest --output --derived-lock
--converter-commit --dry-run; crates/sllm-core/src/gguf_convert.rs.)
"""
from __future__ import annotations

import json
import os
import sys

from .common import CliError, StrictParser, emit, run_main

KINDS = ("random-llama", "hf-llama", "hf-qwen35", "mixed-precision")


def _hf_config(raw: dict, weight_format: str):
    from ..models.config import ModelConfig
    if raw.get("model_type") not in ("llama", "mistral", "qwen2", "qwen3"):
        raise CliError(f"unsupported model_type {raw.get('model_type')!r} for kind hf-llama")
    heads = raw["num_attention_heads"]
    hd = raw.get("head_dim") or raw["hidden_size"] // heads
    return ModelConfig(name=raw.get("_name_or_path") or raw["model_type"], family="llama", n_layers=raw["num_hidden_layers"],
                       d_model=raw["hidden_size"], n_heads=heads, n_kv_heads=raw.get("num_key_value_heads", heads),
                       head_dim=hd, ffn=raw["intermediate_size"], vocab=raw["vocab_size"],
                       rope_theta=float(raw.get("rope_theta", 10000.0)), rms_eps=float(raw.get("rms_norm_eps", 1e-5)),
                       tie_embeddings=bool(raw.get("tie_word_embeddings", False)), weight_format=weight_format,
                       kv_format="fp8" if weight_format == "fp8" else "bf16",
                       max_context=min(int(raw.get("max_position_embeddings", 8192)), 131072))


BENCH_WORDS = ("alpha", "beta", "gamma", "delta", "omega", "sigma", "kappa", "theta", "lambda", "zeta")


def _synthetic_tokenizer(vocab_size: int) -> str:
    """`tokenizers` JSON of a whitespace word-level vocabulary: id i is the word `w<i>`, except that the first ids
    after 0 are the words the serving load generator writes its prompts with; unknown text maps to id 0."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    vocab = {f"w{i}": i for i in range(vocab_size)}
    for j, word in enumerate(BENCH_WORDS, start=1):
        if j < vocab_size:
            del vocab[f"w{j}"]
            vocab[word] = j
    tk = Tokenizer(models.WordLevel(vocab, unk_token="w0"))
    tk.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    return tk.to_str()


def _load_hf(cache, cfg):
    """Reads the safetensors shards through the verified descriptors and assembles LlamaWeights on the CPU."""
    import torch
    from safetensors import safe_open
    from ..models.llama import LayerWeights, LlamaWeights
    from ..ops.core import LinearWeight
    names = [p for p in cache.fds if p.endswith(".safetensors")]
    tensors = {}
    for n in sorted(names):
        with safe_open(os.path.join(cache.root, n), framework="pt") as f:
            for k in f.keys():
                tensors[k] = f.get_tensor(k)
    dt = torch.bfloat16

    def get(name):
        if name not in tensors:
            raise CliError(f"checkpoint lacks tensor {name}")
        return tensors.pop(name).to(dt)

    def lin(w):
        return LinearWeight.from_dense(w.float() if cfg.weight_format == "fp8" else w.contiguous(),
                                       "fp8" if cfg.weight_format == "fp8" else "dense")

    layers = []
    for i in range(cfg.n_layers):
        p = f"model.layers.{i}."
        layers.append(LayerWeights(
            attn_norm=get(p + "input_layernorm.weight"),
            qkv=lin(torch.cat([get(p + "self_attn.q_proj.weight"), get(p + "self_attn.k_proj.weight"),
                               get(p + "self_attn.v_proj.weight")], dim=0)),
            o=lin(get(p + "self_attn.o_proj.weight")),
            mlp_norm=get(p + "post_attention_layernorm.weight"),
            gate_up=lin(torch.cat([get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")], dim=0)),
            down=lin(get(p + "mlp.down_proj.weight"))))
    embed = get("model.embed_tokens.weight")
    head = embed if cfg.tie_embeddings else get("lm_head.weight")
    leftover = [k for k in tensors if not k.endswith("rotary_emb.inv_freq")]
    if leftover:
        raise CliError(f"unconsumed tensors in the checkpoint (unknown policy is reject): {leftover[:4]}")
    return LlamaWeights(embed, layers, get("model.norm.weight"), lin(head), 0)


def _hf_qwen35_config(raw: dict):
    """Model configuration of a Qwen3.5 text decoder (fields as crates/sllm-core/src/model.rs:1138-1260 and
    qwen35_moe.rs:1177-1189 read them)."""
    from ..models.config import ModelConfig
    text = dict(raw.get("text_config") or raw)
    mt = text.get("model_type")
    if mt not in ("qwen3_5_text", "qwen3_5_moe_text"):
        raise CliError(f"unsupported model_type {mt!r} for kind hf-qwen35")
    rp = text.get("rope_parameters") or {}
    hd = int(text["head_dim"])
    ghd = int(text["linear_key_head_dim"])
    if int(text["linear_value_head_dim"]) != ghd:
        raise CliError("gated-delta-net key and value head widths differ")
    sparse = mt == "qwen3_5_moe_text"
    return ModelConfig(
        name=raw.get("_name_or_path") or mt, family="qwen35", n_layers=int(text["num_hidden_layers"]),
        d_model=int(text["hidden_size"]), n_heads=int(text["num_attention_heads"]),
        n_kv_heads=int(text["num_key_value_heads"]), head_dim=hd,
        ffn=int(text["moe_intermediate_size"] if sparse else text["intermediate_size"]), vocab=int(text["vocab_size"]),
        rope_theta=float(rp.get("rope_theta", text.get("rope_theta", 1e7))),
        rotary_dim=int(round(hd * float(rp.get("partial_rotary_factor", text.get("partial_rotary_factor", 0.25))))),
        rms_eps=float(text.get("rms_norm_eps", 1e-6)), norm_offset_one=True, weight_format="bf16", kv_format="bf16",
        qk_norm=True, full_attention_interval=int(text.get("full_attention_interval", 4)),
        gdn_heads=int(text["linear_num_value_heads"]), gdn_qk_heads=int(text["linear_num_key_heads"]), gdn_head_dim=ghd,
        gdn_conv_kernel=int(text["linear_conv_kernel_dim"]), attn_output_gate=bool(text.get("attn_output_gate", True)),
        tie_embeddings=bool(raw.get("tie_word_embeddings", text.get("tie_word_embeddings", False))),
        n_experts=int(text["num_experts"]) if sparse else 0, top_k=int(text["num_experts_per_tok"]) if sparse else 0,
        expert_ffn=int(text["moe_intermediate_size"]) if sparse else 0,
        shared_expert_ffn=int(text.get("shared_expert_intermediate_size", 0)) if sparse else 0,
        expert_format="mxfp4", max_context=min(int(text.get("max_position_embeddings", 8192)), 131072))


def _load_hf_qwen35(cache, cfg):
    """Qwen35Weights on the CPU from the verified safetensors shards, and the names left unconsumed on purpose.

    Source layout (crates/sllm-core/src/model.rs:1406-1540): per layer `input_layernorm`, `post_attention_layernorm`,
    the MLP, and either `linear_attn.{in_proj_qkv,in_proj_z,in_proj_b,in_proj_a,conv1d,A_log,dt_bias,norm,out_proj}` or
    `self_attn.{q_proj,k_proj,v_proj,o_proj,q_norm,k_norm}`, where q_proj holds [query | output gate] per head
    (native/hip/src/attention_preprocess_kernel.hip.cpp:131-135).  Sparse MLP (qwen35_moe.rs:1576-1624): `mlp.gate`
    (router), `mlp.shared_expert_gate`, `mlp.shared_expert.*`, and per expert three packed U8 matrices with U8 E8M0
    scales per 32 inputs."""
    import numpy as np
    import torch
    from safetensors import safe_open
    from ..models.qwen35 import Qwen35Layer, Qwen35Weights
    from ..ops.core import LinearWeight
    from ..ops.w4 import W4Weight
    tensors = {}
    for n in sorted(p for p in cache.fds if p.endswith(".safetensors")):
        with safe_open(os.path.join(cache.root, n), framework="pt") as f:
            for k in f.keys():
                tensors[k] = f.get_tensor(k)
    root = "model.language_model." if any(k.startswith("model.language_model.") for k in tensors) else "model."
    bf = torch.bfloat16

    def get(name, dtype=bf, shape=None):
        if name not in tensors:
            raise CliError(f"checkpoint lacks tensor {name}")
        t = tensors.pop(name)
        if shape is not None and tuple(t.shape) != tuple(shape):
            raise CliError(f"{name}: shape {tuple(t.shape)} differs from the expected {tuple(shape)}")
        return t.to(dtype) if dtype is not None else t

    dense = lambda w: LinearWeight("dense", w.contiguous())
    # --weight-format fp8: projections are quantised to E4M3 with one fp32 scale per 1 x 128 block (the reference's FP8
    # plan takes them from a sidecar instead: gguf_convert.rs:253-329); the router stays bf16
    lin = (lambda w: LinearWeight.from_dense(w.float().contiguous(), "fp8")) if cfg.weight_format == "fp8" else dense
    d, hd, hq, hkv = cfg.d_model, cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
    ghd, vh, qh = cfg.gdn_head_dim, cfg.gdn_heads, cfg.gdn_qk_heads
    width = (2 * qh + vh) * ghd
    E, F, fs = cfg.n_experts, cfg.expert_ffn, cfg.shared_expert_ffn

    def experts(p, stems, n, k):
        """[E, len(stems) * n, k] routed matrices from packed values [n, k / 2] and scales [n, k / 32]."""
        vals = np.empty((E, len(stems) * n, k // 2), dtype=np.uint8)
        scs = np.empty((E, len(stems) * n, k // 32), dtype=np.uint8)
        for e in range(E):
            for j, stem in enumerate(stems):
                base = f"{p}mlp.experts.{e}.{stem}"
                vals[e, j * n:(j + 1) * n] = get(base + ".weight", None, (n, k // 2)).numpy()
                scs[e, j * n:(j + 1) * n] = get(base + ".weight_scale", None, (n, k // 32)).numpy()
        return W4Weight.from_file_layout("mxfp4", vals, scs, k, None, "cpu")

    layers = []
    for i in range(cfg.n_layers):
        p = f"{root}layers.{i}."
        common = dict(in_norm=get(p + "input_layernorm.weight", shape=(d,)),
                      mlp_norm=get(p + "post_attention_layernorm.weight", shape=(d,)))
        if E:
            router = get(p + "mlp.gate.weight", shape=(E, d))
            if fs:
                router = torch.cat([router, get(p + "mlp.shared_expert_gate.weight", shape=(1, d)),
                                    torch.zeros((7, d), dtype=bf)], dim=0)
                common.update(
                    shared_gate_up=lin(torch.cat([get(p + "mlp.shared_expert.gate_proj.weight", shape=(fs, d)),
                                                  get(p + "mlp.shared_expert.up_proj.weight", shape=(fs, d))], dim=0)),
                    shared_down=lin(get(p + "mlp.shared_expert.down_proj.weight", shape=(d, fs))))
            common.update(router=dense(router), exp_gate_up=experts(p, ("gate_proj", "up_proj"), F, d),
                          exp_down=experts(p, ("down_proj",), d, F))
        else:
            f = cfg.ffn
            common.update(gate_up=lin(torch.cat([get(p + "mlp.gate_proj.weight", shape=(f, d)),
                                                 get(p + "mlp.up_proj.weight", shape=(f, d))], dim=0)),
                          down=lin(get(p + "mlp.down_proj.weight", shape=(d, f))))
        if (i + 1) % cfg.full_attention_interval == 0:
            a = p + "self_attn."
            gate = None
            if cfg.attn_output_gate:
                packed = get(a + "q_proj.weight", shape=(2 * hq * hd, d)).view(hq, 2, hd, d)
                wq, gate = packed[:, 0].reshape(hq * hd, d), lin(packed[:, 1].reshape(hq * hd, d))
            else:
                wq = get(a + "q_proj.weight", shape=(hq * hd, d))
            qkv = torch.cat([wq, get(a + "k_proj.weight", shape=(hkv * hd, d)), get(a + "v_proj.weight", shape=(hkv * hd, d))])
            layers.append(Qwen35Layer("full", qkv=lin(qkv), gate=gate, o=lin(get(a + "o_proj.weight", shape=(d, hq * hd))),
                                      q_norm=get(a + "q_norm.weight", shape=(hd,)), k_norm=get(a + "k_norm.weight", shape=(hd,)),
                                      **common))
        else:
            a = p + "linear_attn."
            w_loc = torch.cat([get(a + "in_proj_qkv.weight", shape=(width, d)), get(a + "in_proj_z.weight", shape=(vh * ghd, d)),
                               get(a + "in_proj_b.weight", shape=(vh, d)), get(a + "in_proj_a.weight", shape=(vh, d))], dim=0)
            w_in = torch.zeros(((w_loc.shape[0] + 7) // 8 * 8, d), dtype=bf)
            w_in[:w_loc.shape[0]] = w_loc
            layers.append(Qwen35Layer(
                "gdn", in_proj=lin(w_in),
                conv_w=get(a + "conv1d.weight", shape=(width, 1, cfg.gdn_conv_kernel)).reshape(width, cfg.gdn_conv_kernel).contiguous(),
                a_log=get(a + "A_log", torch.float32, (vh,)), dt_bias=get(a + "dt_bias", shape=(vh,)),
                out_norm=get(a + "norm.weight", torch.float32, (ghd,)), out_proj=lin(get(a + "out_proj.weight", shape=(d, vh * ghd))),
                **common))
    embed = get(root + "embed_tokens.weight", shape=(cfg.vocab, d))
    head = embed if cfg.tie_embeddings else get("lm_head.weight", shape=(cfg.vocab, d))
    final = get(root + "norm.weight", shape=(d,))
    unconsumed = sorted(k for k in tensors if k.startswith(("model.visual.", "mtp.")))
    leftover = [k for k in tensors if k not in unconsumed and not k.endswith("rotary_emb.inv_freq")]
    if leftover:
        raise CliError(f"unconsumed tensors in the checkpoint (unknown policy is reject): {leftover[:4]}")
    head_w = LinearWeight("dense", head) if cfg.tie_embeddings else lin(head)
    return Qwen35Weights(embed, layers, final, head_w, 0), unconsumed


def _write_lock(path: str, doc: dict) -> None:
    tmp = path + ".tmp"
    with open(tmp, "w", encoding="utf-8") as f:
        json.dump(doc, f, sort_keys=True, indent=1)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def main(argv=None) -> int:
    def go():
        p = StrictParser(prog="sllm-convert-gguf")
        p.add_argument("--kind", required=True, choices=KINDS)
        p.add_argument("--lock")
        p.add_argument("--cache")
        p.add_argument("--artifact", help="named shape for random-llama (tiny-llama, llama3-8b, llama-draft, ...)")
        p.add_argument("--manifest", help="optional JSON overriding fields of the model configuration")
        p.add_argument("--output", required=True)
        p.add_argument("--derived-lock", required=True)
        p.add_argument("--converter-commit", default="unknown")
        p.add_argument("--weight-format", choices=("fp32", "bf16", "fp8", "nvfp4", "mxfp4"), default="bf16")
        p.add_argument("--seed", type=int, default=0)
        p.add_argument("--layers", type=int, default=None)
        p.add_argument("--synthetic-tokenizer", action="store_true",
                       help="random-llama: embed a word-level tokenizer in which every id decodes to a visible word "
                            "(serving benchmarks of random weights then stream one text delta per token)")
        p.add_argument("--with-vision", choices=("tiny", "qwen"), default=None,
                       help="random-llama: add a seeded vision tower (tiny: 2 blocks of width 64; qwen: 24 blocks of "
                            "width 1024) whose merger projects to the model width, and 3-axis rotary sections")
        p.add_argument("--with-mtp", action="store_true",
                       help="random-llama: add a seeded multi-token-prediction component (mtp.* tensors)")
        p.add_argument("--dry-run", action="store_true")
        a = p.parse_args(sys.argv[1:] if argv is None else argv)
        import torch
        from ..formats import model_lock as ML
        from ..models import config as MC
        from ..models import loader
        from ..models.llama import init_random_weights
        overrides = {}
        if a.manifest:
            with open(a.manifest, "r", encoding="utf-8") as f:
                overrides = json.load(f)
            if not isinstance(overrides, dict):
                raise CliError("--manifest must hold a JSON object")
        fps, tokenizer_json, chat_template = [], None, None
        named = dict(MC.NAMED)
        from ..models import moe as _moe
        from ..models import qwen35 as _q35
        named.update({"tiny-moe": _moe.tiny_moe, "tiny-shared-moe": _moe.tiny_shared_moe, "tiny-qwen35": _q35.tiny_qwen35,
                      "tiny-qwen35-moe": _q35.tiny_qwen35_moe})
        if a.kind == "random-llama":
            if a.artifact not in named:
                raise CliError(f"--artifact must be one of {sorted(named)}")
            cfg = named[a.artifact]()
            if cfg.family in ("moe", "qwen35"):
                ok = ("bf16", "fp32", "fp8") if cfg.family == "qwen35" else ("bf16", "fp32")
                if a.weight_format not in ok:
                    raise CliError("the mixture-of-experts family keeps bf16 attention (experts are MXFP4); the hybrid "
                                   "family takes bf16, fp32 or fp8 projections")
                if a.with_vision or a.with_mtp:
                    raise CliError("--with-vision / --with-mtp apply to the dense decoder family")
            cfg.weight_format = a.weight_format
            if a.weight_format != "fp8" and cfg.kv_format == "fp8":
                cfg.kv_format = "bf16"
            if a.weight_format == "fp32":
                cfg.kv_format = "fp32"
        else:
            if not (a.lock and a.cache):
                raise CliError(f"kind {a.kind} needs --lock and --cache")
            try:
                lock = ML.read_model_lock(a.lock)
                cache = lock.verify_cache(a.cache)
            except (OSError, ML.ModelLockError) as exc:
                raise CliError(f"source verification failed: {exc}", 3) from None
            fps = [lock.fingerprint]
            raw_cfg = json.loads(cache.read("config.json", 1 << 20))
            if a.kind == "mixed-precision":
                text = dict(raw_cfg.get("text_config") or raw_cfg)
                text.setdefault("model_type", "llama")
                if text["model_type"] not in ("llama", "mistral", "qwen2", "qwen3"):
                    text["model_type"] = "llama"          # the decoder stack of a multimodal wrapper
                cfg = _hf_config(text, "mixed-fp8-nvfp4")
                cfg.kv_format, cfg.tie_embeddings = "fp8-static", True
            elif a.kind == "hf-qwen35":
                if a.weight_format not in ("bf16", "fp8"):
                    raise CliError("kind hf-qwen35 writes bf16 projections or quantises them to block-scaled FP8 "
                                   "(routed experts keep their MXFP4 encoding)")
                cfg = _hf_qwen35_config(raw_cfg)
                cfg.weight_format = a.weight_format
            else:
                cfg = _hf_config(raw_cfg, a.weight_format)
            if "tokenizer.json" in cache.fds:
                tokenizer_json = cache.read("tokenizer.json").decode("utf-8")
            if "chat_template.jinja" in cache.fds:
                chat_template = cache.read("chat_template.jinja", 64 << 10).decode("utf-8")
        if a.layers:
            cfg.n_layers = a.layers
        for k, v in overrides.items():
            if k not in cfg.to_dict():
                raise CliError(f"unknown configuration field {k!r} in --manifest")
            setattr(cfg, k, v)
        plan = {"kind": a.kind, "model": cfg.name, "layers": cfg.n_layers, "weight_format": cfg.weight_format,
                "output": a.output, "derived_lock": a.derived_lock, "source_lock_fingerprints": fps}
        if a.dry_run:
            emit({"dry_run": True, **plan})
            return 0
        if a.kind == "hf-qwen35" or (a.kind == "random-llama" and cfg.family in ("moe", "qwen35")):
            from ..models import family_io
            dev = "cuda" if torch.cuda.is_available() else "cpu"
            extra = {}
            if a.kind == "hf-qwen35":
                w, unconsumed = _load_hf_qwen35(cache, cfg)
                cache.close()
                plan["known_unconsumed_tensors"] = len(unconsumed)
                extra = {"known_unconsumed": unconsumed, "source_fingerprints": tuple(fps)}
            elif cfg.family == "moe":
                w = _moe.init_random_moe_weights(cfg, dev, seed=a.seed)
            else:
                w = _q35.init_random_qwen35_weights(cfg, dev, seed=a.seed)
            if a.synthetic_tokenizer:
                if a.kind != "random-llama":
                    raise CliError("--synthetic-tokenizer applies to kind random-llama")
                tokenizer_json = _synthetic_tokenizer(cfg.vocab)
            dl = family_io.export_family_gguf(cfg, w, a.output, tokenizer_json=tokenizer_json, chat_template=chat_template,
                                              converter_args={"kind": a.kind, "commit": a.converter_commit, "seed": a.seed,
                                                              "weight_format": a.weight_format}, **extra)
            _write_lock(a.derived_lock, dl)
            emit({"written": True, **plan, "size_bytes": dl["output"]["size_bytes"], "sha256": dl["output"]["sha256"],
                  "fingerprint": dl["fingerprint"]})
            return 0
        if a.kind == "random-llama":
            dev = "cuda" if torch.cuda.is_available() else "cpu"
            w = init_random_weights(cfg, dev, seed=a.seed)
        elif a.kind == "mixed-precision":
            from ..formats import quantized_model as QM
            try:
                header, _ = QM.read_safetensors_header(os.path.join(cache.root, "model.safetensors"))
                prefix = "model.language_model" if any(n.startswith("model.language_model.") for n in header) else "model"
                geo = QM.ModelGeometry(cfg.n_layers, cfg.d_model, cfg.q_size, cfg.kv_size, cfg.ffn, cfg.vocab, prefix)
                qm = QM.open_mixed_precision_checkpoint(cache.root, geo)
                w, kv_scales = QM.load_resident(qm, cfg, "cpu")
            except (OSError, QM.QuantizedModelError) as exc:
                raise CliError(f"quantised checkpoint rejected: {exc}", 3) from None
            cfg.kv_static_scales = [[float(k), float(v)] for k, v in kv_scales]
            plan["recipe"] = qm.recipe.to_dict()
            plan["recipe_digest"] = qm.digest
            cache.close()
        else:
            w = _load_hf(cache, cfg)
            cache.close()
        if a.synthetic_tokenizer:
            if a.kind != "random-llama":
                raise CliError("--synthetic-tokenizer applies to kind random-llama")
            tokenizer_json = _synthetic_tokenizer(cfg.vocab)
        vision = None
        if a.with_vision:
            if a.kind != "random-llama":
                raise CliError("--with-vision applies to kind random-llama")
            from dataclasses import asdict
            from ..models import vision_tower as VT
            vc = VT.tiny_vision() if a.with_vision == "tiny" else VT.VisionConfig()
            vc.out_hidden = cfg.d_model
            pairs = (cfg.rotary_dim or cfg.head_dim) // 2
            cfg.vision = asdict(vc)
            cfg.mrope_sections = [pairs // 4, (pairs - pairs // 4) // 2]
            cfg.image_token_id = cfg.vocab - 1
            vision = VT.init_random_vision_weights(vc, dev, seed=a.seed + 2,
                                                   dtype=torch.float32 if cfg.weight_format == "fp32" else torch.bfloat16)
        mtp = None
        if a.with_mtp:
            if a.kind != "random-llama":
                raise CliError("--with-mtp applies to kind random-llama")
            from ..models.mtp import init_random_mtp_weights
            mtp = init_random_mtp_weights(cfg, dev, seed=a.seed + 1)
        dl = loader.export_llama_gguf(cfg, w, a.output, tokenizer_json=tokenizer_json, chat_template=chat_template,
                                      source_fingerprints=tuple(fps), mtp=mtp, vision=vision,
                                      converter_args={"kind": a.kind, "commit": a.converter_commit, "seed": a.seed,
                                                      "weight_format": a.weight_format})
        _write_lock(a.derived_lock, dl)
        emit({"written": True, **plan, "size_bytes": dl["output"]["size_bytes"], "sha256": dl["output"]["sha256"],
              "fingerprint": dl["fingerprint"]})
        return 0
    return run_main(go)


if __name__ == "__main__":
    sys.exit(main())
