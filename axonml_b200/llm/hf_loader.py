"""HuggingFace checkpoint loading (crates/axonml-llm/src/hf_loader.rs:33-333, tokenizer.rs:26-461,
state_dict.rs:74-127): ``HFLoader.from_local(path)`` reads ``config.json``, single or sharded
(``model.safetensors.index.json``) safetensors in F32/F16/BF16, weight-name mappers, and
``HFTokenizer`` (tokenizer.json byte-level BPE).  ``HFLoader.new(model_id)`` resolves a model id in
the local cache directory; there is no network on this machine, so ``download_file`` raises unless
the file is already cached."""
from __future__ import annotations

import json
import os

import torch

from ..serialize.codec import safetensors_loads


class HFLoader:
    def __init__(self, path: str, model_id: str | None = None):
        self.path, self.model_id = path, model_id
        self._tensors = None

    @classmethod
    def new(cls, model_id: str, cache_dir: str | None = None):
        cache = cache_dir or os.path.join(os.path.expanduser("~"), ".axonml", "hub", model_id.replace("/", "--"))
        return cls(cache, model_id)

    @classmethod
    def from_local(cls, path: str): return cls(path)

    def download_file(self, filename: str) -> str:
        p = os.path.join(self.path, filename)
        if not os.path.exists(p):
            raise FileNotFoundError(f"{filename} is not in {self.path} and no network is available to fetch it")
        return p

    def load_config(self) -> dict:
        with open(self.download_file("config.json")) as f:
            return json.load(f)

    def _files(self):
        idx = os.path.join(self.path, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx) as f:
                return sorted(set(json.load(f)["weight_map"].values()))
        return [f for f in sorted(os.listdir(self.path)) if f.endswith(".safetensors")]

    def load_tensors(self) -> dict:
        if self._tensors is None:
            out = {}
            for fn in self._files():
                with open(os.path.join(self.path, fn), "rb") as f:
                    t, _ = safetensors_loads(f.read())
                out.update(t)
            self._tensors = out
        return self._tensors

    def tensor_names(self): return list(self.load_tensors())
    def get_tensor(self, name: str): return self.load_tensors().get(name)
    def get_as_tensor(self, name: str, dtype=torch.float32):
        t = self.get_tensor(name)
        return None if t is None else t.to(dtype)


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


class LoadStateDict:
    """Mixin: ``load_state_dict_from(tensors, strict)`` with shape checks and a report."""

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


class HFTokenizer:
    """Byte-level BPE from a ``tokenizer.json`` (vocab + merges)."""

    def __init__(self, vocab: dict, merges: list, special: dict | None = None):
        self.vocab, self.special = vocab, special or {}
        self.inv = {v: k for k, v in vocab.items()}
        self.ranks = {tuple(m.split(" ")) if isinstance(m, str) else tuple(m): i for i, m in enumerate(merges)}
        bs = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
        cs, n = bs[:], 0
        for b in range(256):
            if b not in bs:
                bs.append(b)
                cs.append(256 + n)
                n += 1
        self.byte_enc = dict(zip(bs, map(chr, cs)))
        self.byte_dec = {v: k for k, v in self.byte_enc.items()}

    @classmethod
    def from_directory(cls, path: str):
        with open(os.path.join(path, "tokenizer.json")) as f:
            j = json.load(f)
        special = {t["content"]: t["id"] for t in j.get("added_tokens", [])}
        return cls(j["model"]["vocab"], j["model"].get("merges", []), special)

    @classmethod
    def from_pretrained(cls, model_id: str): return cls.from_directory(HFLoader.new(model_id).path)

    def _bpe(self, word):
        w = list(word)
        while len(w) > 1:
            pairs = [(self.ranks.get((a, b), 1 << 30), i) for i, (a, b) in enumerate(zip(w, w[1:]))]
            r, i = min(pairs)
            if r == 1 << 30:
                break
            w[i:i + 2] = [w[i] + w[i + 1]]
        return w

    def encode(self, text: str) -> list:
        import re
        ids = []
        for piece in re.findall(r"'s|'t|'re|'ve|'m|'ll|'d| ?\w+| ?[^\s\w]+|\s+(?!\S)|\s+", text):
            tok = "".join(self.byte_enc[b] for b in piece.encode())
            for t in self._bpe(tok):
                if t in self.vocab:
                    ids.append(self.vocab[t])
                else:
                    ids.extend(self.vocab.get(c, 0) for c in t)
        return ids

    def decode(self, ids) -> str:
        s = "".join(self.inv.get(int(i), "") for i in ids)
        return bytes(self.byte_dec.get(c, ord("?")) for c in s).decode("utf-8", "replace")

    def vocab_size(self) -> int: return len(self.vocab)
