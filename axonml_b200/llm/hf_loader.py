"""HuggingFace checkpoint loading.

Parity: crates/axonml-llm/src/hf_loader.rs:33-333 (``HFLoader::new(model_id)`` with a cache
directory per model, ``from_local``, ``download_file`` / ``download_file_if_exists``,
``load_config``, ``load_tensors`` over a single file or the shards named by
``model.safetensors.index.json``, F32 / F16 / BF16 payloads, ``get_tensor`` / ``get_as_tensor`` /
``tensor_names``), :352-460 (weight-name mappers), :484-571 (``load_llama_from_hf``,
``load_mistral_from_hf`` and their config parsers), state_dict.rs (``LoadStateDict``,
``LoadResult``, ``map_hf_to_axonml`` / ``map_axonml_to_hf``, ``load_with_mapping``) and
tokenizer.rs:26-461 (``HFTokenizer`` from ``tokenizer.json`` or ``vocab.json`` + ``merges.txt``,
``SpecialTokens``, ``encode`` / ``encode_with_options`` / ``decode`` / ``decode_with_options``).

Files missing from the model's directory are fetched from the hub endpoint
(``AXONML_HUB_ENDPOINT``, default huggingface.co); without a network that raises ``NetworkError``
naming the file, and everything already on disk keeps working."""
from __future__ import annotations

import dataclasses
import json
import os
import re

import torch

from ..hub.download import NetworkError as _HubNetworkError
from ..hub.download import fetch, hub_cache_root, repo_url
from ..serialize.codec import safetensors_loads
from . import error as E


class HFLoader:
    def __init__(self, path: str, model_id: str | None = None):
        self.path, self.model_id = path, model_id
        self._tensors = None

    @classmethod
    def new(cls, model_id: str, cache_dir: str | None = None):
        """Loader for a hub model id (``org/name``); its files live in a cache directory of their own."""
        cache = cache_dir or os.path.join(hub_cache_root(), "hf", model_id.replace("/", "--"))
        os.makedirs(cache, exist_ok=True)
        return cls(cache, model_id)

    @classmethod
    def from_local(cls, path: str):
        if not os.path.isdir(path):
            raise E.ModelNotFound(path)
        return cls(path)

    def download_file(self, filename: str) -> str:
        """Path of ``filename`` in the model directory, fetched from the hub when absent."""
        p = os.path.join(self.path, filename)
        if os.path.exists(p):
            return p
        if self.model_id is None:
            raise E.ModelNotFound(f"{filename} is not in {self.path}")
        try:
            return fetch(repo_url(self.model_id, filename), p)
        except _HubNetworkError as e:
            raise E.NetworkError(f"{filename} of {self.model_id}: {e}") from e

    def download_file_if_exists(self, filename: str) -> bool:
        """True when the file is (now) in the model directory; False when the hub does not have it."""
        try:
            self.download_file(filename)
            return True
        except (E.NetworkError, E.ModelNotFound):
            return False

    def load_config(self) -> dict:
        try:
            with open(self.download_file("config.json")) as f:
                return json.load(f)
        except ValueError as e:
            raise E.ParseError(f"config.json: {e}") from e

    def _files(self):
        idx = os.path.join(self.path, "model.safetensors.index.json")
        if not os.path.exists(idx) and self.model_id is not None and not os.path.exists(os.path.join(self.path, "model.safetensors")):
            self.download_file_if_exists("model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx) as f:
                return sorted(set(json.load(f)["weight_map"].values()))
        local = [f for f in sorted(os.listdir(self.path)) if f.endswith(".safetensors")]
        return local or ["model.safetensors"]

    def load_tensors(self) -> dict:
        if self._tensors is None:
            out = {}
            for fn in self._files():
                with open(self.download_file(fn), "rb") as f:
                    try:
                        t, _ = safetensors_loads(f.read())
                    except (ValueError, KeyError) as e:
                        raise E.UnsupportedFormat(f"{fn}: {e}") from e
                out.update(t)
            self._tensors = out
        return self._tensors

    def cache_dir(self) -> str:
        """Directory the model's files are (or will be) in."""
        return self.path

    @property
    def tensors(self) -> dict:
        """``{name: tensor}`` of everything loaded so far (empty before ``load_tensors``)."""
        return self._tensors or {}

    def print_tensor_info(self, limit: int | None = None) -> None:
        """One line per tensor: name, stored dtype, shape, element count."""
        names = self.tensor_names()
        for n in names[:limit]:
            i = self.tensor_info(n)
            print(f"{n:60s} {i.dtype:5s} {str(i.shape):24s} {i.numel():>12,d}")
        total = sum(t.numel() for t in self.load_tensors().values())
        print(f"{len(names)} tensors, {total:,d} elements")

    def tensor_names(self): return list(self.load_tensors())
    def get_tensor(self, name: str): return self.load_tensors().get(name)

    def get_as_tensor(self, name: str, dtype=torch.float32):
        t = self.get_tensor(name)
        return None if t is None else t.to(dtype)

    def tensor_info(self, name: str):
        """``TensorInfo`` of one tensor (its stored dtype and shape), or ``None``."""
        t = self.get_tensor(name)
        if t is None:
            return None
        names = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.float64: "F64", torch.int64: "I64",
                 torch.int32: "I32", torch.int8: "I8", torch.uint8: "U8", torch.bool: "BOOL"}
        return TensorInfo(list(t.shape), t, names.get(t.dtype, str(t.dtype)))

    def require(self, name: str, dtype=torch.float32) -> torch.Tensor:
        t = self.get_as_tensor(name, dtype)
        if t is None:
            raise E.WeightNotFound(name)
        return t


def map_llama_weights(sd: dict) -> dict:
    """HF LLaMA names -> this package's names (drops the ``model.`` prefix; hf_loader.rs:352-405)."""
    return {(k[6:] if k.startswith("model.") else k): v for k, v in sd.items()}


def map_llama_weights_alt(sd: dict) -> dict:
    """The reference's second scheme (state_dict.rs:74-127): ``self_attn`` -> ``attention``,
    ``input_layernorm`` -> ``input_norm``, ``post_attention_layernorm`` -> ``post_attn_norm``."""
    out = {}
    for k, v in map_llama_weights(sd).items():
        out[k.replace("self_attn", "attention").replace("input_layernorm", "input_norm")
             .replace("post_attention_layernorm", "post_attn_norm")] = v
    return out


def map_gpt2_weights(sd: dict) -> dict:
    """HF GPT-2 names -> GPT2LMHead names; HF stores Conv1D weights as [in, out], so they are transposed."""
    out = {}
    for k, v in sd.items():
        k = k.removeprefix("transformer.")
        if k == "wte.weight": out["transformer.wte.wte.weight"] = v
        elif k == "wpe.weight": out["transformer.wte.wpe.weight"] = v
        elif k.startswith("ln_f."): out["transformer." + k] = v
        elif k.startswith("h."):
            _, i, rest = k.split(".", 2)
            rest = (rest.replace("ln_1", "ln1").replace("ln_2", "ln2").replace("attn.c_attn", "attention.c_attn")
                    .replace("attn.c_proj", "attention.c_proj").replace("mlp.c_fc", "ffn.fc1").replace("mlp.c_proj", "ffn.fc2"))
            if rest.endswith("weight") and v.dim() == 2 and ("c_attn" in rest or "c_proj" in rest or "fc1" in rest or "fc2" in rest):
                v = v.t().contiguous()
            out[f"transformer.blocks.{i}.{rest}"] = v
    return out



@dataclasses.dataclass
class TensorInfo:
    """One tensor of a checkpoint as the loader reports it (hf_loader.rs:46-53)."""
    shape: list
    data: torch.Tensor
    dtype: str                     # the stored type: "F32", "F16", "BF16", ...

    def numel(self) -> int: return self.data.numel()


class WeightMapper:
    """Names of a family's checkpoint -> names of this package's model (hf_loader.rs:343-349)."""

    def __init__(self, num_layers: int):
        self.num_layers = num_layers

    @classmethod
    def new(cls, num_layers: int): return cls(num_layers)

    def map_name(self, hf_name: str):
        """The model's name for ``hf_name``, or ``None`` for a tensor the model does not use."""
        raise NotImplementedError

    def expected_weights(self) -> list:
        raise NotImplementedError

    def map_all(self, tensors: dict) -> dict:
        out = {}
        for k, v in tensors.items():
            name = self.map_name(k)
            if name is not None:
                out[name] = v
        return out

    def missing(self, tensors: dict) -> list:
        """Expected names absent from ``tensors`` (after mapping)."""
        have = set(self.map_all(tensors))
        return [w for w in self.expected_weights() if w not in have]


class LLaMAWeightMapper(WeightMapper):
    _PER_LAYER = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj", "mlp.up_proj",
                  "mlp.down_proj", "input_layernorm", "post_attention_layernorm")
    _TOP = ("embed_tokens.weight", "norm.weight")

    def map_name(self, hf_name: str):
        if "rotary_emb.inv_freq" in hf_name:
            return None
        return hf_name.removeprefix("model.")

    def expected_weights(self) -> list:
        return list(self._TOP) + [f"layers.{i}.{n}.weight" for i in range(self.num_layers) for n in self._PER_LAYER]


class MistralWeightMapper(LLaMAWeightMapper):
    """Mistral checkpoints use LLaMA's names."""


class PhiWeightMapper(WeightMapper):
    _PER_LAYER = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.dense", "mlp.fc1", "mlp.fc2", "input_layernorm")

    def map_name(self, hf_name: str):
        if "rotary_emb.inv_freq" in hf_name:
            return None
        return hf_name.removeprefix("model.") if hf_name.startswith("model.") else hf_name.removeprefix("transformer.")

    def expected_weights(self) -> list:
        return (["embed_tokens.weight", "final_layernorm.weight"]
                + [f"layers.{i}.{n}.weight" for i in range(self.num_layers) for n in self._PER_LAYER])


def map_hf_to_axonml(hf_name: str, arch: str) -> str:
    """One HuggingFace tensor name in the reference's alternative naming (state_dict.rs:74-101)."""
    name = hf_name.removeprefix("model.") if hf_name.startswith("model.") else hf_name.removeprefix("transformer.")
    if arch in ("llama", "mistral"):
        return (name.replace("self_attn.", "attention.").replace("input_layernorm", "input_norm")
                .replace("post_attention_layernorm", "post_attn_norm"))
    if arch == "phi":
        return name.replace("self_attn.", "attention.").replace("fc1", "up_proj").replace("fc2", "down_proj")
    return name


def map_axonml_to_hf(axonml_name: str, arch: str) -> str:
    """Inverse of ``map_hf_to_axonml`` (state_dict.rs:104-127)."""
    if arch in ("llama", "mistral"):
        return "model." + (axonml_name.replace("attention.", "self_attn.").replace("input_norm", "input_layernorm")
                           .replace("post_attn_norm", "post_attention_layernorm"))
    if arch == "phi":
        return "model." + axonml_name.replace("attention.", "self_attn.").replace("up_proj", "fc1").replace("down_proj", "fc2")
    return axonml_name


@dataclasses.dataclass
class LoadResult:
    unexpected_keys: list = dataclasses.field(default_factory=list)
    missing_keys: list = dataclasses.field(default_factory=list)
    loaded_count: int = 0
    mismatched_keys: list = dataclasses.field(default_factory=list)

    def is_success(self, strict: bool) -> bool:
        return not strict or not (self.missing_keys or self.mismatched_keys)

    def summary(self) -> str:
        lines = [f"Loaded {self.loaded_count} parameters"]
        for title, keys in (("Missing", self.missing_keys), ("Unexpected", self.unexpected_keys), ("Mismatched", self.mismatched_keys)):
            if keys:
                lines.append(f"{title} keys ({len(keys)}):")
                lines += [f"  - {k}" for k in keys]
        return "\n".join(lines)

    def print_summary(self) -> None:
        print(self.summary())


def load_with_mapping(model, weights: dict, arch: str, strict: bool = False) -> LoadResult:
    """Loads HuggingFace-named ``weights`` into ``model``: the ``model.`` / ``transformer.`` prefix
    is dropped, GPT-2's transposed Conv1D weights are turned, and names the model does not have are
    retried in the reference's alternative scheme."""
    own = {k for k, _ in model.named_parameters()}
    if arch == "bert":
        from .bert import map_bert_weights
        mapped = map_bert_weights(weights, "bert." if any(k.startswith("bert.") for k in own) else "")
    elif arch == "gpt2":
        mapped = map_gpt2_weights(weights)
        if not any(k in own for k in mapped):               # a bare GPT2 without the LM-head wrapper
            mapped = {k.removeprefix("transformer."): v for k, v in mapped.items()}
    else:
        mapped = {}
        for k, v in weights.items():
            plain = k.removeprefix("model.")
            alt = map_hf_to_axonml(k, arch)
            mapped[next((c for c in (k, plain, "model." + plain, alt, "model." + alt) if c in own), alt)] = v
    # tied output head: checkpoints that share it with the embedding store the embedding only
    for head, emb in (("lm_head.weight", "model.embed_tokens.weight"), ("lm_head.weight", "embed_tokens.weight")):
        if head in own and head not in mapped and emb in mapped:
            mapped[head] = mapped[emb]
    r = LoadStateDict.load_state_dict_from(model, mapped, strict=False)
    res = LoadResult(r["unexpected"], r["missing"], len(r["loaded"]), r["mismatched"])
    if not res.is_success(strict):
        raise E.LoadError(res.summary())
    return res


def parse_llama_config_from_json(j: dict):
    from .config import LLaMAConfig
    heads = int(j.get("num_attention_heads", 32))
    return LLaMAConfig(vocab_size=int(j.get("vocab_size", 32000)), hidden_size=int(j.get("hidden_size", 4096)),
                       intermediate_size=int(j.get("intermediate_size", 11008)), num_hidden_layers=int(j.get("num_hidden_layers", 32)),
                       num_attention_heads=heads, num_key_value_heads=int(j.get("num_key_value_heads") or heads),
                       max_position_embeddings=int(j.get("max_position_embeddings", 4096)),
                       rms_norm_eps=float(j.get("rms_norm_eps", 1e-5)), rope_theta=float(j.get("rope_theta", 10000.0)))


def parse_mistral_config(j: dict):
    from .config import MistralConfig
    return MistralConfig(vocab_size=int(j.get("vocab_size", 32000)), hidden_size=int(j.get("hidden_size", 4096)),
                         intermediate_size=int(j.get("intermediate_size", 14336)), num_hidden_layers=int(j.get("num_hidden_layers", 32)),
                         num_attention_heads=int(j.get("num_attention_heads", 32)), num_key_value_heads=int(j.get("num_key_value_heads", 8)),
                         max_position_embeddings=int(j.get("max_position_embeddings", 32768)),
                         rms_norm_eps=float(j.get("rms_norm_eps", 1e-5)), rope_theta=float(j.get("rope_theta", 10000.0)),
                         sliding_window=int(j.get("sliding_window") or 4096))


def _load_from_hf(model_or_path: str, parse):
    loader = HFLoader.from_local(model_or_path) if os.path.isdir(model_or_path) else HFLoader.new(model_or_path)
    cfg = parse(loader.load_config())
    weights = {k: v.float() for k, v in loader.load_tensors().items() if "rotary_emb.inv_freq" not in k}
    return cfg, weights


def load_llama_from_hf(model_id: str):
    """``(LLaMAConfig, {name: fp32 tensor})`` of a hub model id or a local directory, under the
    checkpoint's own names; ``load_with_mapping(model, weights, "llama")`` puts them into a model."""
    return _load_from_hf(model_id, parse_llama_config_from_json)


def load_mistral_from_hf(model_id: str):
    return _load_from_hf(model_id, parse_mistral_config)


class LoadStateDict:
    """Mixin: ``load_state_dict_from(tensors, strict)`` with shape checks and a report."""

    def state_dict_keys(self) -> list:
        return [k for k, _ in self.named_parameters()]

    def load_state_dict_from(self, tensors: dict, strict: bool = False) -> dict:
        own = dict(self.named_parameters())
        report = {"loaded": [], "missing": [], "unexpected": [k for k in tensors if k not in own], "mismatched": []}
        with torch.no_grad():
            for k, p in own.items():
                if k not in tensors:
                    report["missing"].append(k)
                    continue
                t = torch.as_tensor(tensors[k])
                if t.numel() != p.numel():
                    if t.dim() == 2 and p.dim() == 2 and t.shape[1] == p.shape[1] and t.shape[0] < p.shape[0]:
                        p[:t.shape[0]].copy_(t.to(p.dtype))       # padded vocabulary
                        report["loaded"].append(k)
                    else:
                        report["mismatched"].append(k)
                    continue
                p.copy_(t.reshape(p.shape).to(p.dtype))
                report["loaded"].append(k)
        if strict and (report["missing"] or report["mismatched"]):
            raise KeyError(str({k: report[k] for k in ("missing", "mismatched")}))
        return report


@dataclasses.dataclass
class SpecialTokens:
    bos_token: str | None = None
    eos_token: str | None = None
    unk_token: str | None = None
    pad_token: str | None = None
    bos_token_id: int | None = None
    eos_token_id: int | None = None
    unk_token_id: int | None = None
    pad_token_id: int | None = None


def _bytes_to_unicode() -> dict:
    """GPT-2's printable stand-in for every byte value."""
    bs = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    cs, n = bs[:], 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return dict(zip(bs, map(chr, cs)))


_GPT2_SPLIT = re.compile(r"'s|'t|'re|'ve|'m|'ll|'d| ?[^\W\d_]+| ?\d+| ?[^\s\w]+|\s+(?!\S)|\s+")
_TOKEN_NAME = re.compile(r"^(bos|eos|unk|pad)_token$")


class HFTokenizer:
    """BPE tokenizer read from HuggingFace files.  Two vocabularies are recognised: byte-level
    (GPT-2 style: every byte has a printable stand-in, words carry their leading space as ``Ġ``)
    and SentencePiece-style (LLaMA / Mistral: spaces become ``▁``, unknown characters fall back to
    ``<0xNN>`` byte tokens).  Added tokens are matched whole before the text is split."""

    def __init__(self, vocab: dict, merges: list, special: dict | None = None, special_tokens: SpecialTokens | None = None,
                 style: str | None = None, add_prefix_space: bool = True):
        self.vocab = dict(vocab)
        self.added_tokens = dict(special or {})
        self.special = self.added_tokens                      # earlier name, kept
        self.inv = {v: k for k, v in self.vocab.items()}
        self.inv.update({v: k for k, v in self.added_tokens.items()})
        pairs = [tuple(m.split(" ")) if isinstance(m, str) else tuple(m) for m in merges]
        self.ranks = {p: i for i, p in enumerate(pairs) if len(p) == 2}
        self.byte_enc = _bytes_to_unicode()
        self.byte_dec = {v: k for k, v in self.byte_enc.items()}
        if style is None:
            style = "sentencepiece" if any(t.startswith("\u2581") for t in list(self.vocab)[:5000]) or "<0x0A>" in self.vocab else "bytelevel"
        self.style, self.add_prefix_space = style, add_prefix_space
        self._special = special_tokens or SpecialTokens()
        self._added_re = (re.compile("(" + "|".join(re.escape(t) for t in sorted(self.added_tokens, key=len, reverse=True)) + ")")
                          if self.added_tokens else None)
        self._cache: dict[str, list] = {}

    # ------------------------------------------------------------------ loading
    @classmethod
    def from_directory(cls, path: str):
        tj = os.path.join(path, "tokenizer.json")
        if os.path.exists(tj):
            return cls._load_tokenizer_json(tj, path)
        vj = os.path.join(path, "vocab.json")
        if os.path.exists(vj):
            return cls._load_legacy(vj, os.path.join(path, "merges.txt"), path)
        raise E.ModelNotFound("No tokenizer.json or vocab.json found in " + path)

    @classmethod
    def from_pretrained(cls, model_id: str):
        if os.path.isdir(model_id):
            return cls.from_directory(model_id)
        loader = HFLoader.new(model_id)
        if loader.download_file_if_exists("tokenizer.json"):
            loader.download_file_if_exists("tokenizer_config.json")
        else:
            loader.download_file("vocab.json")
            loader.download_file_if_exists("merges.txt")
            loader.download_file_if_exists("special_tokens_map.json")
        return cls.from_directory(loader.path)

    @staticmethod
    def _read_json(path: str) -> dict:
        try:
            with open(path, encoding="utf-8") as f:
                return json.load(f)
        except OSError as e:
            raise E.IoError(str(e)) from e
        except ValueError as e:
            raise E.ParseError(f"{os.path.basename(path)}: {e}") from e

    @classmethod
    def _named_specials(cls, directory: str, lookup) -> SpecialTokens:
        """bos / eos / unk / pad by name from tokenizer_config.json or special_tokens_map.json."""
        st = SpecialTokens()
        for fn in ("special_tokens_map.json", "tokenizer_config.json"):
            p = os.path.join(directory, fn)
            if not os.path.exists(p):
                continue
            try:
                j = cls._read_json(p)
            except E.LLMError:
                continue
            for key, val in j.items():
                if not _TOKEN_NAME.match(key) or val is None:
                    continue
                content = val.get("content") if isinstance(val, dict) else val
                if isinstance(content, str):
                    setattr(st, key, content)
                    setattr(st, key + "_id", lookup(content))
        return st

    @classmethod
    def _load_tokenizer_json(cls, path: str, directory: str):
        j = cls._read_json(path)
        model = j.get("model") or {}
        vocab = {t: int(i) for t, i in (model.get("vocab") or {}).items()}
        added, flagged = {}, SpecialTokens()
        for t in j.get("added_tokens") or []:
            content, tid = t.get("content"), t.get("id")
            if not isinstance(content, str) or tid is None:
                continue
            added[content] = int(tid)
            if t.get("special"):
                low = content.lower()
                kind = ("bos" if "bos" in low or low in ("<s>", "<|begin_of_text|>") else
                        "eos" if "eos" in low or low in ("</s>", "<|end_of_text|>", "<|endoftext|>") else
                        "unk" if "unk" in low else "pad" if "pad" in low else None)
                if kind and getattr(flagged, kind + "_token") is None:
                    setattr(flagged, kind + "_token", content)
                    setattr(flagged, kind + "_token_id", int(tid))
        lookup = lambda tok: added.get(tok, vocab.get(tok))
        named = cls._named_specials(directory, lookup)
        for f in dataclasses.fields(SpecialTokens):               # names given explicitly win over guesses
            if getattr(named, f.name) is not None:
                setattr(flagged, f.name, getattr(named, f.name))
        pre = json.dumps(j.get("pre_tokenizer") or {}) + json.dumps(j.get("decoder") or {})
        style = "bytelevel" if "ByteLevel" in pre else "sentencepiece" if ("Metaspace" in pre or model.get("byte_fallback")) else None
        norm = json.dumps(j.get("normalizer") or {})
        prefix = "Prepend" in norm or '"add_prefix_space": true' in pre or '"prepend_scheme": "always"' in pre or '"prepend_scheme": "first"' in pre
        return cls(vocab, model.get("merges") or [], added, flagged, style, add_prefix_space=prefix or style != "sentencepiece")

    @classmethod
    def _load_legacy(cls, vocab_path: str, merges_path: str, directory: str):
        vocab = {t: int(i) for t, i in cls._read_json(vocab_path).items()}
        merges = []
        if os.path.exists(merges_path):
            with open(merges_path, encoding="utf-8") as f:
                for line in f:
                    parts = line.rstrip("\n").split(" ")
                    if len(parts) == 2 and not line.startswith("#version"):
                        merges.append((parts[0], parts[1]))
        st = cls._named_specials(directory, vocab.get)
        added = {getattr(st, k + "_token"): getattr(st, k + "_token_id") for k in ("bos", "eos", "unk", "pad")
                 if getattr(st, k + "_token_id") is not None}
        return cls(vocab, merges, added, st)

    # ------------------------------------------------------------------ encoding
    def _bpe(self, symbols: list) -> list:
        w = list(symbols)
        while len(w) > 1:
            best, at = None, -1
            for i in range(len(w) - 1):
                r = self.ranks.get((w[i], w[i + 1]))
                if r is not None and (best is None or r < best):
                    best, at = r, i
            if best is None:
                break
            first, second = w[at], w[at + 1]
            out, i = [], 0
            while i < len(w):                                # merge every occurrence of the best pair
                if i < len(w) - 1 and w[i] == first and w[i + 1] == second:
                    out.append(first + second)
                    i += 2
                else:
                    out.append(w[i])
                    i += 1
            w = out
        return w

    def _word_ids(self, word: str) -> list:
        hit = self._cache.get(word)
        if hit is not None:
            return hit
        ids = []
        for t in self._bpe(list(word)):
            tid = self.vocab.get(t)
            if tid is not None:
                ids.append(tid)
                continue
            for ch in t:                                      # a merge result that is not a token: spell it out
                cid = self.vocab.get(ch)
                if cid is not None:
                    ids.append(cid)
                elif self.style == "sentencepiece":
                    fallback = [self.vocab.get(f"<0x{b:02X}>") for b in ch.encode("utf-8")]
                    ids += fallback if all(f is not None for f in fallback) else [self._special.unk_token_id or 0]
                else:
                    ids.append(self._special.unk_token_id or 0)
        if len(self._cache) < 50_000:
            self._cache[word] = ids
        return ids

    def _encode_plain(self, text: str, first: bool) -> list:
        if not text:
            return []
        ids = []
        if self.style == "sentencepiece":
            s = text.replace(" ", "\u2581")
            if first and self.add_prefix_space and not s.startswith("\u2581"):
                s = "\u2581" + s
            for piece in re.findall("\u2581*[^\u2581]+|\u2581+$", s):
                ids += self._word_ids(piece)
            return ids
        for piece in _GPT2_SPLIT.findall(text):
            ids += self._word_ids("".join(self.byte_enc[b] for b in piece.encode("utf-8")))
        return ids

    def bpe_encode(self, text: str) -> list:
        """Token ids of ``text`` without BOS / EOS; added tokens inside the text map to their ids."""
        if self._added_re is None:
            return self._encode_plain(text, True)
        ids, first = [], True
        for part in self._added_re.split(text):
            if part in self.added_tokens:
                ids.append(self.added_tokens[part])
            elif part:
                ids += self._encode_plain(part, first)
            first = False if part else first
        return ids

    def encode(self, text: str) -> list:
        """BOS (when the tokenizer defines one) followed by the tokens of ``text``."""
        return self.encode_with_options(text, add_bos=True, add_eos=False)

    def encode_with_options(self, text: str, add_bos: bool = True, add_eos: bool = False, max_length: int | None = None) -> list:
        ids = []
        if add_bos and self._special.bos_token_id is not None:
            ids.append(self._special.bos_token_id)
        ids += self.bpe_encode(text)
        if add_eos and self._special.eos_token_id is not None:
            ids.append(self._special.eos_token_id)
        return ids[:max_length] if max_length else ids

    def encode_batch(self, texts, add_bos: bool = True, add_eos: bool = False, pad_to: int | None = None):
        """Lists of ids; with ``pad_to`` every row is cut or right-padded with the pad (else EOS, else 0) id."""
        rows = [self.encode_with_options(t, add_bos, add_eos) for t in texts]
        if pad_to is None:
            return rows
        pad = self._special.pad_token_id
        pad = pad if pad is not None else self._special.eos_token_id if self._special.eos_token_id is not None else 0
        return [r[:pad_to] + [pad] * (pad_to - len(r)) for r in rows]

    # ------------------------------------------------------------------ decoding
    def decode(self, ids) -> str:
        return self.decode_with_options(ids, True)

    def decode_with_options(self, ids, skip_special: bool = True) -> str:
        skip = {self._special.bos_token_id, self._special.eos_token_id, self._special.pad_token_id} - {None} if skip_special else set()
        out, buf = [], bytearray()

        def flush():
            if buf:
                out.append(buf.decode("utf-8", "replace"))
                buf.clear()

        for i in ids:
            i = int(i)
            if i in skip:
                continue
            tok = self.inv.get(i)
            if tok is None:
                continue
            if tok in self.added_tokens:
                flush()
                out.append(tok)
            elif self.style == "sentencepiece":
                if len(tok) == 6 and tok.startswith("<0x") and tok.endswith(">"):
                    try:
                        buf.append(int(tok[3:5], 16))
                        continue
                    except ValueError:
                        pass
                flush()
                out.append(tok.replace("\u2581", " "))
            else:
                for c in tok:
                    b = self.byte_dec.get(c)
                    if b is None:
                        buf.extend(c.encode("utf-8"))
                    else:
                        buf.append(b)
        flush()
        text = "".join(out)
        if self.style == "sentencepiece" and self.add_prefix_space and text.startswith(" "):
            text = text[1:]
        return text

    # ------------------------------------------------------------------ lookups
    def vocab_size(self) -> int: return len(self.inv)
    def special_tokens(self) -> SpecialTokens: return self._special
    def bos_token_id(self): return self._special.bos_token_id
    def eos_token_id(self): return self._special.eos_token_id
    def pad_token_id(self): return self._special.pad_token_id
    def id_to_token(self, i: int): return self.inv.get(int(i))
    def token_to_id(self, token: str): return self.added_tokens.get(token, self.vocab.get(token))
