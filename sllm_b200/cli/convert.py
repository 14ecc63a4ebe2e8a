"""`sllm-convert-gguf`: writes a GGUF file plus its derived lock.

Kinds:
  random-llama   seeded random-init weights of a named shape (`--artifact llama3-8b`), for benchmarks and tests; the
                 mixture-of-experts (`moe-120b`, `qwen35-moe`, `tiny-moe`, `tiny-shared-moe`) and hybrid
                 (`qwen35-hybrid`, `tiny-qwen35`) shapes are written through models/family_io.py with MXFP4 experts
  hf-llama       a Llama-style Hugging Face checkpoint (config.json + safetensors) from a directory that is first
                 verified against its model lock (`--lock lock.json --cache DIR`)
  mixed-precision  a compressed-tensors checkpoint with FP8 channel-scaled attention projections, NVFP4 MLP
                 projections and per-layer static FP8 KV scales (formats/quantized_model.py); same lock verification.
                 The file keeps the FP8 matrices block-scaled, the NVFP4 matrices as GGML type-40 blocks with their
                 outer scales, and the KV scales in the model configuration
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

KINDS = ("random-llama", "hf-llama", "mixed-precision")


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
        named.update({"tiny-moe": _moe.tiny_moe, "tiny-shared-moe": _moe.tiny_shared_moe, "tiny-qwen35": _q35.tiny_qwen35})
        if a.kind == "random-llama":
            if a.artifact not in named:
                raise CliError(f"--artifact must be one of {sorted(named)}")
            cfg = named[a.artifact]()
            if cfg.family in ("moe", "qwen35"):
                if a.weight_format not in ("bf16", "fp32"):
                    raise CliError("the mixture-of-experts and hybrid families keep bf16 attention (experts are MXFP4)")
                if a.with_vision or a.with_mtp:
                    raise CliError("--with-vision / --with-mtp apply to the dense decoder family")
            cfg.weight_format = a.weight_format
            if a.weight_format != "fp8" and cfg.kv_format == "fp8":
                cfg.kv_format = "bf16"
            if a.weight_format == "fp32":
                cfg.kv_format = "fp32"
        else:
            if not (a.lock and a.cache):
                raise CliError("kind hf-llama needs --lock and --cache")
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
        if a.kind == "random-llama" and cfg.family in ("moe", "qwen35"):
            from ..models import family_io
            dev = "cuda" if torch.cuda.is_available() else "cpu"
            if cfg.family == "moe":
                w = _moe.init_random_moe_weights(cfg, dev, seed=a.seed)
            else:
                w = _q35.init_random_qwen35_weights(cfg, dev, seed=a.seed)
            if a.synthetic_tokenizer:
                tokenizer_json = _synthetic_tokenizer(cfg.vocab)
            dl = family_io.export_family_gguf(cfg, w, a.output, tokenizer_json=tokenizer_json, chat_template=chat_template,
                                              converter_args={"kind": a.kind, "commit": a.converter_commit, "seed": a.seed,
                                                              "weight_format": a.weight_format})
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
