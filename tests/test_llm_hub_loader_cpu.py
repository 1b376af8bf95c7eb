"""Model hubs, HuggingFace checkpoint loading, tokenizers and the generic transformer stacks.

Mirrors the reference's tests in crates/axonml-llm/src/hub.rs (registry contents, cache paths,
architecture and parameter-budget filters), state_dict.rs (name mapping, LoadResult), tokenizer.rs
and crates/axonml-vision/src/hub.rs (registry, save / load round trip); downloads run against a
local HTTP server."""
import hashlib
import http.server
import json
import os
import threading

import pytest
import torch

from axonml_b200 import llm, vision
from axonml_b200.hub import download as dl
from axonml_b200.llm import error as E
from axonml_b200.llm import hub as lhub
from axonml_b200.serialize.codec import safetensors_dumps


@pytest.fixture()
def hub_server(tmp_path, monkeypatch):
    """Serves tmp_path/site as the hub endpoint; the cache lives in tmp_path/cache."""
    site = tmp_path / "site"
    site.mkdir()

    class H(http.server.SimpleHTTPRequestHandler):
        def __init__(self, *a, **kw):
            super().__init__(*a, directory=str(site), **kw)

        def log_message(self, *a):
            pass

    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    monkeypatch.setenv("AXONML_HUB_ENDPOINT", f"http://127.0.0.1:{srv.server_address[1]}")
    monkeypatch.setenv("AXONML_HUB_CACHE", str(tmp_path / "cache"))
    yield site
    srv.shutdown()
    srv.server_close()


def _put(site, repo, filename, data: bytes):
    d = site / repo / "resolve" / "main"
    d.mkdir(parents=True, exist_ok=True)
    (d / filename).write_bytes(data)


# ---------------------------------------------------------------------------------------------- hubs
def test_llm_registry_contents_and_filters():
    reg = llm.llm_registry()
    for name in ("bert-base-uncased", "gpt2", "distilbert-base-uncased", "llama-2-7b", "mistral-7b", "phi-2", "qwen-7b"):
        assert name in reg
    g = reg["gpt2"]
    assert (g.vocab_size, g.hidden_size, g.num_layers, g.num_heads, g.max_seq_len, g.architecture) == (50257, 768, 12, 12, 1024, "GPT2")
    assert g.url.endswith("/axonml-ml/gpt2/resolve/main/model.safetensors") and g.params_str() == "124.0M"
    assert reg["llama-2-7b"].url.startswith("https://huggingface.co/meta-llama/Llama-2-7b-hf/")
    assert {m.name for m in lhub.models_by_architecture("bert")} == {"bert-tiny", "bert-mini", "bert-base-uncased", "bert-base-cased",
                                                                     "bert-large-uncased"}
    small = lhub.models_by_max_params(100_000_000)
    assert [m.num_parameters for m in small] == sorted(m.num_parameters for m in small) and small[0].name == "bert-tiny"
    assert all(m.num_parameters <= 100_000_000 for m in small) and "gpt2" not in {m.name for m in small}
    assert lhub.model_info("nope") is None and len(lhub.list_models()) == len(reg) == 23
    # sizes are consistent with the architecture: 12 h^2 per layer plus embeddings, within 25 %
    for m in reg.values():
        if m.architecture in ("BERT", "GPT2", "RoBERTa"):
            est = 12 * m.hidden_size ** 2 * m.num_layers + m.vocab_size * m.hidden_size
            assert 0.75 < est / m.num_parameters < 1.25, m.name


def test_llm_weights_download_cache_and_errors(hub_server, capsys):
    blob = safetensors_dumps({"w": torch.arange(6.0).view(2, 3)})
    _put(hub_server, "axonml-ml/bert-tiny", "model.safetensors", blob)
    assert lhub.cache_dir().endswith(os.path.join("cache", "llm")) and not lhub.is_cached("bert-tiny")
    p = llm.download_llm_weights("bert-tiny")
    assert p == lhub.cached_path("bert-tiny") and open(p, "rb").read() == blob and lhub.is_cached("bert-tiny")
    assert "Downloading bert-tiny (17.0 MB, 4.4M parameters)" in capsys.readouterr().out
    _put(hub_server, "axonml-ml/bert-tiny", "model.safetensors", b"changed")
    assert open(llm.download_llm_weights("bert-tiny", quiet=True), "rb").read() == blob          # cached copy wins
    assert open(llm.download_llm_weights("bert-tiny", force=True, quiet=True), "rb").read() == b"changed"
    with pytest.raises(dl.ModelNotFound) as e:
        llm.download_llm_weights("not-a-model")
    assert str(e.value) == "Model not found: not-a-model" and isinstance(e.value, KeyError)
    with pytest.raises(dl.NetworkError) as e:
        llm.download_llm_weights("gpt2", quiet=True)                                         # the server has no such file
    assert "HTTP 404" in str(e.value) and not lhub.is_cached("gpt2")
    assert not os.path.exists(lhub.cached_path("gpt2") + ".part")                            # nothing half-written is left


def test_download_checks_the_checksum_and_reports_an_unreachable_host(hub_server, tmp_path, monkeypatch):
    _put(hub_server, "org/repo", "f.bin", b"payload")
    url = dl.repo_url("org/repo", "f.bin")
    good = hashlib.sha256(b"payload").hexdigest()
    dest = str(tmp_path / "out" / "f.bin")
    seen = []
    assert dl.fetch(url, dest, good.upper(), progress=lambda done, total: seen.append((done, total))) == dest
    assert seen[-1] == (7, 7) and dl.sha256_file(dest) == good
    with pytest.raises(dl.InvalidFormat):
        dl.fetch(url, dest + "2", "0" * 64)
    assert not os.path.exists(dest + "2") and not os.path.exists(dest + "2.part")
    monkeypatch.setenv("AXONML_HUB_ENDPOINT", "http://127.0.0.1:9")                              # discard port: refused
    with pytest.raises(dl.NetworkError) as e:
        dl.fetch(dl.repo_url("org/repo", "f.bin"), dest + "3", timeout=2.0)
    assert e.value.kind == "NetworkError" and str(e.value).startswith("Network error: ")
    assert dl.format_params(1_558_000_000) == "1.6B" and dl.format_params(950) == "950"


def test_vision_registry_download_and_weight_file_round_trip(hub_server):
    reg = vision.model_registry()
    assert len(reg) == 22 and {"resnet18", "vgg16_bn", "mobilenet_v3_large", "efficientnet_b2", "vit_b_16", "swin_t", "convnext_small"} <= set(reg)
    r = reg["resnet18"]
    assert (r.num_classes, r.input_size, r.dataset, r.accuracy, r.size_bytes) == (1000, (224, 224), "ImageNet-1K", 69.76, 44_700_000)
    assert reg["efficientnet_b2"].input_size == (260, 260) and vision.model_info("resnet999") is None
    assert r.url.endswith("/axonml-ml/resnet18-imagenet/resolve/main/resnet18.safetensors")
    assert len(vision.list_models()) == 22 and vision.cache_dir().endswith(os.path.join("cache", "weights"))
    state = {"conv1.weight": torch.randn(4, 3, 3, 3), "fc.bias": torch.randn(10), "scale": torch.tensor(2.5)}
    _put(hub_server, "axonml-ml/resnet18-imagenet", "resnet18.safetensors", safetensors_dumps(state))
    assert not vision.is_cached("resnet18")
    p = vision.download_weights("resnet18", quiet=True)
    assert vision.is_cached("resnet18")
    back = vision.load_state_dict(p)                                       # a SafeTensors file is recognised
    assert set(back) == set(state) and all(torch.equal(back[k], state[k]) for k in state)
    path = os.path.join(vision.cache_dir(), "own.bin")
    vision.hub.save_state_dict(state, path)                                # the hub's own u32-count format
    own = vision.load_state_dict(path)
    assert all(torch.equal(own[k], state[k]) and own[k].shape == state[k].shape for k in state)
    with open(path, "wb") as f:
        f.write(b"\x05\x00\x00\x00\xff\xff\xff\xff")
    with pytest.raises(vision.HubError):
        vision.load_state_dict(path)
    with pytest.raises(vision.HubError):
        vision.download_weights("resnet999")


# ---------------------------------------------------------------------------------------------- loader
def _tiny_llama_dir(path, sharded=False, dtype=torch.bfloat16, tied=False):
    cfg = llm.LLaMAConfig.tiny()
    torch.manual_seed(1)
    ref = llm.LLaMAForCausalLM(cfg)
    sd = {k: v.detach().to(dtype) for k, v in ref.named_parameters()}
    if tied:
        with torch.no_grad():
            ref.lm_head.weight.copy_(ref.model.embed_tokens.weight.to(dtype).float())
        sd.pop("lm_head.weight")
    sd["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(4)
    os.makedirs(path, exist_ok=True)
    json.dump({"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
               "num_hidden_layers": cfg.num_hidden_layers, "num_attention_heads": cfg.num_attention_heads,
               "num_key_value_heads": cfg.num_key_value_heads, "max_position_embeddings": cfg.max_position_embeddings,
               "rms_norm_eps": cfg.rms_norm_eps, "rope_theta": cfg.rope_theta, "sliding_window": 16}, open(os.path.join(path, "config.json"), "w"))
    if sharded:
        names = sorted(sd)
        half = len(names) // 2
        parts = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
        for fn, ks in parts.items():
            open(os.path.join(path, fn), "wb").write(safetensors_dumps({k: sd[k] for k in ks}))
        json.dump({"weight_map": {k: fn for fn, ks in parts.items() for k in ks}}, open(os.path.join(path, "model.safetensors.index.json"), "w"))
    else:
        open(os.path.join(path, "model.safetensors"), "wb").write(safetensors_dumps(sd))
    return cfg, ref


@pytest.mark.parametrize("sharded,dtype", [(False, torch.bfloat16), (True, torch.float16), (False, torch.float32)])
def test_llama_checkpoint_directory_loads_into_the_model(tmp_path, sharded, dtype):
    cfg, ref = _tiny_llama_dir(str(tmp_path / "ck"), sharded, dtype)
    got_cfg, weights = llm.load_llama_from_hf(str(tmp_path / "ck"))
    assert got_cfg == cfg and all(v.dtype == torch.float32 for v in weights.values())
    assert not any("inv_freq" in k for k in weights) and len(weights) == len(list(ref.named_parameters()))
    model = llm.LLaMAForCausalLM(got_cfg)
    res = llm.load_with_mapping(model, weights, "llama", strict=True)
    assert res.loaded_count == len(weights) and not res.missing_keys and not res.unexpected_keys and res.is_success(True)
    ids = torch.randint(0, cfg.vocab_size, (2, 9))
    want = {k: v.detach().to(dtype).float() for k, v in ref.named_parameters()}
    assert all(torch.equal(p.detach(), want[k]) for k, p in model.named_parameters())
    with torch.no_grad():
        ref.load_state_dict({k: v for k, v in want.items()}, strict=False)
        assert torch.allclose(model(ids), ref(ids), atol=1e-5)
    # the bare decoder takes the same weights without the "model." prefix, and the alternative names too
    bare = llm.LLaMA(got_cfg)
    r2 = llm.load_with_mapping(bare, weights, "llama")
    assert r2.loaded_count == len(weights) - 1 and r2.unexpected_keys == ["lm_head.weight"] and not r2.missing_keys
    alt = {llm.map_hf_to_axonml(k, "llama"): v for k, v in weights.items()}
    assert "layers.0.attention.q_proj.weight" in alt and "layers.1.post_attn_norm.weight" in alt
    assert {llm.map_axonml_to_hf(k, "llama") for k in alt if k != "lm_head.weight"} == {k for k in weights if k != "lm_head.weight"}


def test_tied_head_missing_weights_and_mistral_config(tmp_path):
    cfg, ref = _tiny_llama_dir(str(tmp_path / "tied"), tied=True, dtype=torch.float32)
    _, weights = llm.load_llama_from_hf(str(tmp_path / "tied"))
    assert "lm_head.weight" not in weights
    model = llm.LLaMAForCausalLM(cfg)
    res = llm.load_with_mapping(model, weights, "llama", strict=True)
    assert torch.equal(model.lm_head.weight, model.model.embed_tokens.weight) and not res.missing_keys
    del weights["model.norm.weight"]
    lenient = llm.load_with_mapping(llm.LLaMAForCausalLM(cfg), weights, "llama")
    assert lenient.missing_keys == ["model.norm.weight"] and lenient.is_success(False) and not lenient.is_success(True)
    assert "Missing keys (1):\n  - model.norm.weight" in lenient.summary()
    with pytest.raises(E.LoadError):
        llm.load_with_mapping(llm.LLaMAForCausalLM(cfg), weights, "llama", strict=True)
    mcfg, _ = llm.load_mistral_from_hf(str(tmp_path / "tied"))
    assert isinstance(mcfg, llm.MistralConfig) and mcfg.sliding_window == 16 and mcfg.hidden_size == cfg.hidden_size
    assert llm.map_hf_to_axonml("model.layers.0.self_attn.q_proj.weight", "llama") == "layers.0.attention.q_proj.weight"
    assert llm.map_hf_to_axonml("model.layers.3.mlp.fc1.bias", "phi") == "layers.3.mlp.up_proj.bias"
    assert llm.map_axonml_to_hf("layers.3.mlp.down_proj.bias", "phi") == "model.layers.3.mlp.fc2.bias"
    assert llm.map_hf_to_axonml("transformer.h.0.ln_1.weight", "gpt2") == "h.0.ln_1.weight"
    r = llm.LoadResult(loaded_count=10)
    assert r.is_success(True)
    r.missing_keys.append("x")
    assert not r.is_success(True) and r.is_success(False)


def test_loader_fetches_missing_files_from_the_hub(hub_server, tmp_path):
    cfg, _ = _tiny_llama_dir(str(tmp_path / "src"), dtype=torch.float32)
    for fn in ("config.json", "model.safetensors"):
        _put(hub_server, "acme/tiny-llama", fn, open(tmp_path / "src" / fn, "rb").read())
    loader = llm.HFLoader.new("acme/tiny-llama")
    assert loader.path.endswith(os.path.join("hf", "acme--tiny-llama")) and os.listdir(loader.path) == []
    assert loader.load_config()["hidden_size"] == cfg.hidden_size
    assert len(loader.tensor_names()) == 22 and loader.get_tensor("nope") is None
    assert loader.get_as_tensor("model.norm.weight").dtype == torch.float32
    assert sorted(os.listdir(loader.path)) == ["config.json", "model.safetensors"]
    assert not loader.download_file_if_exists("tokenizer.json")
    with pytest.raises(E.NetworkError) as e:
        loader.download_file("tokenizer.json")
    assert "tokenizer.json of acme/tiny-llama" in str(e.value)
    with pytest.raises(E.WeightNotFound):
        loader.require("nope")
    with pytest.raises(E.ModelNotFound):
        llm.HFLoader.from_local(str(tmp_path / "absent"))
    with pytest.raises(E.ModelNotFound):
        llm.HFLoader.from_local(str(tmp_path)).download_file("config.json")
    (tmp_path / "src" / "config.json").write_text("{broken")
    with pytest.raises(E.ParseError):
        llm.HFLoader.from_local(str(tmp_path / "src")).load_config()
    cfg2, weights = llm.load_llama_from_hf("acme/tiny-llama")                                # by model id, through the cache
    assert cfg2 == cfg and len(weights) == 21


def test_gpt2_checkpoint_names_and_transposed_weights():
    cfg = llm.GPT2Config.tiny()
    torch.manual_seed(0)
    ref = llm.GPT2LMHead(cfg)
    hf = {}
    for k, v in ref.named_parameters():
        if not k.startswith("transformer."):
            continue
        k2 = k.removeprefix("transformer.")
        if k2 == "wte.wte.weight": hf["transformer.wte.weight"] = v.detach()
        elif k2 == "wte.wpe.weight": hf["transformer.wpe.weight"] = v.detach()
        elif k2.startswith("ln_f."): hf["transformer." + k2] = v.detach()
        else:
            _, i, rest = k2.split(".", 2)
            rest = (rest.replace("ln1", "ln_1").replace("ln2", "ln_2").replace("attention.c_attn", "attn.c_attn")
                    .replace("attention.c_proj", "attn.c_proj").replace("ffn.fc1", "mlp.c_fc").replace("ffn.fc2", "mlp.c_proj"))
            hf[f"transformer.h.{i}.{rest}"] = v.detach().t().contiguous() if rest.endswith("weight") and v.dim() == 2 else v.detach()
    model = llm.GPT2LMHead(cfg)
    res = llm.load_with_mapping(model, hf, "gpt2", strict=True)
    assert res.loaded_count == len(hf) and not res.unexpected_keys
    ids = torch.randint(0, cfg.vocab_size, (2, 7))
    model.eval(); ref.eval()
    with torch.no_grad():
        assert torch.allclose(model(ids), ref(ids), atol=1e-5)
    assert model.state_dict_keys()[0] == "transformer.wte.wte.weight"


# ---------------------------------------------------------------------------------------------- tokenizers
def _bytelevel_dir(path):
    os.makedirs(path, exist_ok=True)
    enc = llm.HFTokenizer({}, []).byte_enc
    base = [enc[b] for b in range(256)]
    merges = [("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o"), ("Ġ", "w"), ("o", "r"), ("Ġw", "or"), ("Ġwor", "l"),
              ("Ġworl", "d"), ("Ġ", "hello")]
    toks = base + [a + b for a, b in merges]
    vocab = {t: i for i, t in enumerate(toks)}
    tj = {"model": {"type": "BPE", "vocab": vocab, "merges": [f"{a} {b}" for a, b in merges]},
          "pre_tokenizer": {"type": "ByteLevel", "add_prefix_space": False},
          "added_tokens": [{"id": len(toks), "content": "<|endoftext|>", "special": True}, {"id": len(toks) + 1, "content": "<|user|>", "special": False}]}
    json.dump(tj, open(os.path.join(path, "tokenizer.json"), "w"))
    return vocab, len(toks)


def test_byte_level_tokenizer(tmp_path):
    vocab, n = _bytelevel_dir(str(tmp_path / "tok"))
    tok = llm.HFTokenizer.from_directory(str(tmp_path / "tok"))
    assert tok.style == "bytelevel" and tok.vocab_size() == n + 2
    assert tok.eos_token_id() == n and tok.bos_token_id() is None and tok.special_tokens().eos_token == "<|endoftext|>"
    ids = tok.encode("hello world")
    assert ids == [vocab["hello"], vocab["Ġworld"]]                      # no BOS is defined, none is added
    assert tok.encode(" hello") == [vocab["Ġhello"]] and tok.decode(ids) == "hello world"
    assert tok.encode_with_options("hello", add_bos=True, add_eos=True) == [vocab["hello"], n]
    mixed = tok.encode("hello<|user|> world<|endoftext|>")
    assert mixed == [vocab["hello"], n + 1, vocab["Ġworld"], n]           # added tokens are matched whole
    assert tok.decode(mixed) == "hello<|user|> world" and tok.decode_with_options(mixed, skip_special=False).endswith("<|endoftext|>")
    text = "naïve café 日本語\n\ttabs  and   spaces 123!?"
    assert tok.decode(tok.encode(text)) == text                             # any text survives through the byte alphabet
    assert tok.id_to_token(vocab["hello"]) == "hello" and tok.token_to_id("<|user|>") == n + 1 and tok.token_to_id("zzz") is None
    assert tok.encode_batch(["hello", "hello world hello"], pad_to=3) == [[vocab["hello"], n, n], [vocab["hello"], vocab["Ġworld"], vocab["Ġhello"]]]
    assert tok.encode_with_options("hello world hello", max_length=2) == [vocab["hello"], vocab["Ġworld"]]


def test_sentencepiece_style_tokenizer_with_byte_fallback(tmp_path):
    d = tmp_path / "sp"
    d.mkdir()
    specials = ["<unk>", "<s>", "</s>"]
    bytes_ = [f"<0x{b:02X}>" for b in range(256)]
    chars = ["▁", "t", "h", "e", "c", "a", "s", "i", "o", "n", "m"]
    merges = [("▁", "t"), ("h", "e"), ("▁t", "he"), ("a", "t"), ("▁", "c"), ("▁c", "at"), ("▁", "s"), ("▁s", "at"),
              ("o", "n"), ("▁", "on")]
    toks = specials + bytes_ + chars + [a + b for a, b in merges]
    vocab = {t: i for i, t in enumerate(toks)}
    json.dump({"model": {"type": "BPE", "vocab": vocab, "merges": [list(m) for m in merges], "byte_fallback": True},
               "normalizer": {"type": "Sequence", "normalizers": [{"type": "Prepend", "prepend": "▁"}]},
               "decoder": {"type": "Sequence", "decoders": [{"type": "Replace"}, {"type": "ByteFallback"}]},
               "added_tokens": [{"id": 0, "content": "<unk>", "special": True}, {"id": 1, "content": "<s>", "special": True},
                                {"id": 2, "content": "</s>", "special": True}]}, open(d / "tokenizer.json", "w"))
    json.dump({"bos_token": {"content": "<s>"}, "eos_token": "</s>", "unk_token": "<unk>", "pad_token": None}, open(d / "tokenizer_config.json", "w"))
    tok = llm.HFTokenizer.from_directory(str(d))
    st = tok.special_tokens()
    assert tok.style == "sentencepiece" and (st.bos_token_id, st.eos_token_id, st.unk_token_id, st.pad_token_id) == (1, 2, 0, None)
    ids = tok.encode("the cat sat on the mat")
    assert ids[0] == 1 and [tok.id_to_token(i) for i in ids[1:]] == ["▁the", "▁cat", "▁sat", "▁on", "▁the", "▁", "m", "at"]
    assert tok.decode(ids) == "the cat sat on the mat"
    assert tok.encode_with_options("the", add_bos=False, add_eos=True) == [vocab["▁the"], 2]
    odd = tok.encode_with_options("the é", add_bos=False)
    assert [tok.id_to_token(i) for i in odd] == ["▁the", "▁", "<0xC3>", "<0xA9>"] and tok.decode(odd) == "the é"
    assert tok.decode_with_options([1] + odd + [2], skip_special=False) == "<s> the é</s>"      # the word keeps its space after a special token


def test_legacy_vocab_and_merges_files(tmp_path):
    d = tmp_path / "legacy"
    d.mkdir()
    enc = llm.HFTokenizer({}, []).byte_enc
    toks = [enc[b] for b in range(256)] + ["ab", "abc", "<|endoftext|>"]
    json.dump({t: i for i, t in enumerate(toks)}, open(d / "vocab.json", "w"))
    (d / "merges.txt").write_text("#version: 0.2\na b\nab c\n")
    json.dump({"bos_token": "<|endoftext|>", "eos_token": "<|endoftext|>", "unk_token": "<|endoftext|>"}, open(d / "special_tokens_map.json", "w"))
    tok = llm.HFTokenizer.from_pretrained(str(d))
    assert tok.bos_token_id() == 258 and tok.eos_token_id() == 258
    assert tok.encode("abc") == [258, 257] and tok.encode_with_options("abcab", add_bos=False) == [257, 256]
    assert tok.decode(tok.encode("abc<|endoftext|>abc")) == "abcabc"
    with pytest.raises(E.ModelNotFound):
        llm.HFTokenizer.from_directory(str(tmp_path))


# ---------------------------------------------------------------------------------------------- layers
def test_llm_errors_carry_the_reference_messages():
    assert str(E.InvalidConfig("heads")) == "Invalid configuration: heads" and isinstance(E.InvalidConfig("x"), (llm.LLMError, ValueError))
    s = E.ShapeMismatch([2, 3], [3, 2])
    assert str(s) == "Shape mismatch: expected [2, 3], got [3, 2]" and (s.expected, s.actual) == ([2, 3], [3, 2])
    assert str(E.WeightNotFound("lm_head.weight")) == "Weight not found: 'lm_head.weight'" or "lm_head.weight" in str(E.WeightNotFound("lm_head.weight"))
    for cls, prefix in ((E.GenerationError, "Generation error"), (E.LoadError, "Model loading error"), (E.IoError, "IO error"),
                        (E.NetworkError, "Network error"), (E.ParseError, "Parse error"), (E.ModelNotFound, "Model not found"),
                        (E.UnsupportedFormat, "Unsupported format"), (E.TensorError, "Tensor error"), (E.CoreError, "Core error"),
                        (E.InvalidInput, "Invalid input")):
        assert issubclass(cls, llm.LLMError) and prefix in str(cls("detail"))


def test_embedding_layers():
    torch.manual_seed(0)
    te = llm.TokenEmbedding(50, 8)
    ids = torch.tensor([[1, 2, 3], [4, 5, 49]])
    assert te.forward_ids(ids).shape == (2, 3, 8) and torch.equal(te(ids)[0, 1], te.embedding.weight[2])
    pe = llm.PositionalEmbedding(16, 8)
    p = pe.forward_positions(5, 2)
    assert p.shape == (2, 5, 8) and torch.equal(p[0], p[1]) and torch.equal(p[0, 3], pe.embedding.weight[3])
    assert torch.equal(pe.forward_positions(2, 1, offset=4)[0, 0], pe.embedding.weight[4])
    with pytest.raises(E.InvalidInput):
        pe.forward_positions(17, 1)
    sp = llm.SinusoidalPositionalEncoding(32, 8)
    e = sp.forward_seq(10)
    assert e.shape == (10, 8) and torch.all(e[0, 0::2] == 0) and torch.all(e[0, 1::2] == 1)
    pos, i = 7, 2
    angle = pos / 10000.0 ** (2 * i / 8)
    assert e[pos, 2 * i].item() == pytest.approx(torch.sin(torch.tensor(angle)).item(), abs=1e-6)
    assert e[pos, 2 * i + 1].item() == pytest.approx(torch.cos(torch.tensor(angle)).item(), abs=1e-6)
    assert not list(sp.parameters()) and torch.equal(sp(torch.zeros(2, 4, 8))[1], e[:4])
    be = llm.BertEmbedding(50, 16, 2, 8, 1e-12, 0.0)
    out = be.forward_with_ids(ids)
    want = torch.nn.functional.layer_norm(be.word_embeddings.weight[ids] + be.position_embeddings.weight[:3] + be.token_type_embeddings.weight[0],
                                          (8,), be.layer_norm.weight, be.layer_norm.bias, 1e-12)
    assert torch.allclose(out, want, atol=1e-5)
    tt = torch.tensor([[0, 0, 1], [1, 1, 1]])
    assert not torch.allclose(be.forward_with_ids(ids, tt), out) and len(list(be.parameters())) == 5


def _ref_attention(m, x, add_mask=None, causal=False):
    B, S, H = x.shape
    h, d = m.num_heads, m.head_dim
    q = torch.nn.functional.linear(x, m.query.weight, m.query.bias).view(B, S, h, d).transpose(1, 2)
    k = torch.nn.functional.linear(x, m.key.weight, m.key.bias).view(B, S, h, d).transpose(1, 2)
    v = torch.nn.functional.linear(x, m.value.weight, m.value.bias).view(B, S, h, d).transpose(1, 2)
    s = q @ k.transpose(-1, -2) / d ** 0.5
    if add_mask is not None:
        s = s + add_mask
    if causal:
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
    o = (torch.softmax(s, -1) @ v).transpose(1, 2).reshape(B, S, H)
    return torch.nn.functional.linear(o, m.out_proj.weight, m.out_proj.bias)


def test_multi_head_self_attention_masks():
    torch.manual_seed(0)
    m = llm.MultiHeadSelfAttention(32, 4, 0.0)
    x = torch.randn(2, 6, 32)
    assert sorted(k for k, _ in m.named_parameters()) == sorted(f"{n}.{p}" for n in ("query", "key", "value", "out_proj") for p in ("weight", "bias"))
    assert torch.allclose(m(x), _ref_attention(m, x), atol=1e-5)
    add = torch.zeros(2, 1, 1, 6)
    add[1, ..., 4:] = float("-inf")                                       # rank 1 hides its last two keys
    got = m.forward_with_mask(x, add)
    assert torch.allclose(got, _ref_attention(m, x, add), atol=1e-5)
    keep = torch.ones(2, 6, dtype=torch.bool)
    keep[1, 4:] = False
    assert torch.allclose(m.forward_with_mask(x, keep), got, atol=1e-6)       # the boolean [batch, key] form says the same
    assert torch.allclose(m.forward_with_mask(x, None, causal=True), _ref_attention(m, x, causal=True), atol=1e-5)
    x2 = x.clone()
    x2[1, 5] += 1.0                                                       # a hidden key does not influence visible rows
    assert torch.allclose(m.forward_with_mask(x2, keep)[1, :4], got[1, :4], atol=1e-6)
    with pytest.raises(ValueError):
        llm.MultiHeadSelfAttention(30, 4)


@pytest.mark.parametrize("pre_norm", [False, True])
def test_transformer_encoder_matches_a_plain_restatement(pre_norm):
    torch.manual_seed(0)
    enc = llm.TransformerEncoder(2, 32, 4, 64, 0.0, 1e-6, "gelu", pre_norm)
    x = torch.randn(2, 5, 32)
    h = x
    for l in enc.layers:
        ln = lambda n, t: torch.nn.functional.layer_norm(t, (32,), n.weight, n.bias, 1e-6)
        ffn = lambda t: torch.nn.functional.linear(torch.nn.functional.gelu(torch.nn.functional.linear(t, l.ffn.fc1.weight, l.ffn.fc1.bias), approximate="tanh"),
                                                   l.ffn.fc2.weight, l.ffn.fc2.bias)
        if pre_norm:
            h = h + _ref_attention(l.attention, ln(l.ln1, h))
            h = h + ffn(ln(l.ln2, h))
        else:
            h = ln(l.ln1, h + _ref_attention(l.attention, h))
            h = ln(l.ln2, h + ffn(h))
    assert torch.allclose(enc(x), h, atol=2e-4)
    keys = [k for k, _ in enc.named_parameters()]
    assert "layers.0.attention.query.weight" in keys and "layers.1.ffn.fc2.bias" in keys and "layers.0.ln2.weight" in keys
    enc(x).sum().backward()
    assert all(p.grad is not None for p in enc.parameters())
    cfg = llm.TransformerConfig(hidden_size=32, num_attention_heads=4, intermediate_size=64, num_layers=3, dropout_prob=0.0)
    assert cfg.head_dim() == 8 and len(llm.TransformerEncoder.from_config(cfg).layers) == 3
    with pytest.raises(E.InvalidConfig):
        llm.TransformerEncoder.from_config(llm.TransformerConfig(hidden_size=30, num_attention_heads=4))
    d = llm.TransformerConfig()
    assert (d.hidden_size, d.num_attention_heads, d.intermediate_size, d.num_layers, d.vocab_size, d.layer_norm_eps) == (768, 12, 3072, 12, 30522, 1e-12)


def test_transformer_decoder_is_causal():
    torch.manual_seed(0)
    dec = llm.TransformerDecoder(2, 32, 4, 16, 0.0, 1e-5, "relu")
    x = torch.randn(1, 8, 32)
    y = dec(x)
    x2 = x.clone()
    x2[0, 5:] += 1.0
    y2 = dec(x2)
    assert torch.allclose(y[0, :5], y2[0, :5], atol=1e-5) and not torch.allclose(y[0, 5:], y2[0, 5:])
    assert "ln_f.weight" in dict(dec.named_parameters()) and dec.layers[0].ffn.fc1.weight.shape == (128, 32)
    with pytest.raises(E.InvalidInput):
        dec(torch.randn(1, 17, 32))
    with pytest.raises(ValueError):
        llm.TransformerDecoder(1, 32, 4, 16, activation="sigmoidish")


def test_flash_attention_config_defaults_and_exports():
    c = llm.FlashAttentionConfig()
    assert (c.block_size_q, c.block_size_kv, c.causal, c.softmax_scale, c.dropout_p) == (64, 64, True, None, 0.0)
    for name in ("RMSNorm", "MultiHeadSelfAttention", "TransformerEncoder", "TransformerDecoder", "TokenEmbedding", "PositionalEmbedding",
                 "BertEmbedding", "GPT2Embedding", "LLMError", "LoadResult", "SpecialTokens", "PretrainedLLM", "llm_registry",
                 "download_llm_weights", "load_llama_from_hf", "load_mistral_from_hf", "TransformerConfig", "FlashAttentionConfig"):
        assert hasattr(llm, name), name
    for name in ("vgg11_bn", "vgg13", "vgg13_bn", "vgg16_bn", "vgg19_bn", "PretrainedModel", "model_registry", "download_weights"):
        assert hasattr(vision, name), name


def test_beam_search_steps_and_search():
    import math
    bs = llm.BeamSearch.new(2, 1.0, True, [3])
    beams = bs.init_beams(torch.tensor([[5, 6]]))
    assert len(beams) == 1 and beams[0].tokens == [5, 6] and beams[0].score == 0.0 and not beams[0].finished
    lp = torch.log(torch.tensor([0.1, 0.6, 0.25, 0.05]))
    beams = bs.expand_beams(beams, [lp])
    assert [b.tokens[-1] for b in beams] == [1, 2] and beams[0].score == pytest.approx(math.log(0.6)) and not any(b.finished for b in beams)
    assert beams[0].normalized_score(1.0) == pytest.approx(math.log(0.6) / 3) and beams[0].normalized_score(0.0) == pytest.approx(math.log(0.6))
    step2 = [torch.log(torch.tensor([0.05, 0.05, 0.1, 0.8])), torch.log(torch.tensor([0.25, 0.25, 0.25, 0.25]))]
    beams = bs.expand_beams(beams, step2)
    assert beams[0].tokens == [5, 6, 1, 3] and beams[0].finished and not bs.should_stop(beams)        # the second beam is still open
    assert bs.best_sequence(beams) == [5, 6, 1, 3]
    kept = bs.expand_beams(beams, [None, torch.log(torch.tensor([0.01, 0.01, 0.01, 0.97]))])
    assert kept[0].tokens == [5, 6, 1, 3] and all(b.finished for b in kept) and bs.should_stop(kept)      # finished beams are carried over
    assert llm.BeamSearch(2).best_sequence([]) is None and llm.BeamSearch(2).best_sequence([llm.Beam.new([1])]) == [1]
    assert not llm.BeamSearch(2, early_stopping=False).should_stop(kept)

    class Chain(torch.nn.Module):            # token t is followed by t+1 with p=0.9, by 0 otherwise; 4 ends the text
        def forward(self, ids):
            nxt = (ids[:, -1] + 1).clamp(max=4)
            logits = torch.full((ids.shape[0], ids.shape[1], 5), math.log(0.1 / 4))
            logits[torch.arange(ids.shape[0]), -1, nxt] = math.log(0.9)
            return logits

    out = llm.BeamSearch(3, 1.0, True).search(Chain(), torch.tensor([[1]]), llm.GenerationConfig(max_new_tokens=8, eos_token_ids=[4]))
    assert out.tolist() == [[1, 2, 3, 4]]


def test_bert_heads_and_published_checkpoint_names():
    cfg = llm.BertConfig(vocab_size=60, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                         max_position_embeddings=16, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    torch.manual_seed(0)
    ref = llm.BertForMaskedLM(cfg).eval()
    keys = [k for k, _ in ref.named_parameters()]
    assert "bert.pooler.dense.weight" in keys and "cls.transform.dense.weight" in keys and "cls.transform.layer_norm.bias" in keys and "cls.bias" in keys
    assert not any("decoder" in k for k in keys) and len(keys) == len(set(keys))          # the projection is the embedding matrix
    inv = {"query": "attention.self.query", "key": "attention.self.key", "value": "attention.self.value", "attn_out": "attention.output.dense",
           "attn_norm": "attention.output.LayerNorm", "intermediate": "intermediate.dense", "output": "output.dense", "out_norm": "output.LayerNorm"}
    hf = {"bert.embeddings.position_ids": torch.arange(16).unsqueeze(0)}
    for k, v in ref.named_parameters():
        if k.startswith("bert.layers."):
            _, _, i, name, leaf = k.split(".")
            hf[f"bert.encoder.layer.{i}.{inv[name]}.{leaf}"] = v.detach()
        elif k.startswith("cls."):
            hf["cls.predictions." + k[4:].replace("layer_norm", "LayerNorm")] = v.detach()
        else:
            hf[k] = v.detach()
    hf["cls.predictions.decoder.weight"] = ref.bert.embeddings.word_embeddings.weight.detach()
    hf["bert.embeddings.LayerNorm.gamma"] = hf.pop("bert.embeddings.LayerNorm.weight")          # the oldest checkpoints' spelling
    hf["bert.embeddings.LayerNorm.beta"] = hf.pop("bert.embeddings.LayerNorm.bias")
    model = llm.BertForMaskedLM(cfg).eval()
    res = llm.load_with_mapping(model, hf, "bert", strict=True)
    assert res.loaded_count == len(keys) and not res.unexpected_keys and not res.missing_keys
    ids = torch.randint(0, 60, (2, 7))
    with torch.no_grad():
        assert torch.allclose(model(ids), ref(ids), atol=1e-5) and model(ids).shape == (2, 7, 60)
    bare = llm.Bert(cfg).eval()
    r2 = llm.load_with_mapping(bare, hf, "bert")
    assert not r2.missing_keys and sorted(r2.unexpected_keys) == sorted(k for k in keys if k.startswith("cls."))
    with torch.no_grad():
        seq, pooled = bare(ids)
        assert torch.allclose(pooled, torch.tanh(torch.nn.functional.linear(seq[:, 0], bare.pooler.dense.weight, bare.pooler.dense.bias)), atol=1e-5)
    pooler = llm.BertPooler.new(8)
    assert pooler(torch.randn(3, 5, 8)).shape == (3, 8)
    head = llm.BertLMPredictionHead(8, 20, activation="relu")                                    # untied: owns its decoder
    assert head(torch.randn(2, 3, 8)).shape == (2, 3, 20) and "decoder.weight" in dict(head.named_parameters())
    t = llm.BertPredictionHeadTransform.new(8, 1e-12, "gelu")
    x = torch.randn(4, 8)
    want = torch.nn.functional.layer_norm(torch.nn.functional.gelu(torch.nn.functional.linear(x, t.dense.weight, t.dense.bias), approximate="tanh"),
                                          (8,), t.layer_norm.weight, t.layer_norm.bias, 1e-12)
    assert torch.allclose(t(x), want, atol=1e-5)


def test_weight_mappers_cover_what_the_models_expect(tmp_path):
    cfg, _ = _tiny_llama_dir(str(tmp_path / "ck"), dtype=torch.bfloat16)
    loader = llm.HFLoader.from_local(str(tmp_path / "ck"))
    m = llm.LLaMAWeightMapper.new(cfg.num_hidden_layers)
    mapped = m.map_all(loader.load_tensors())
    assert m.map_name("model.layers.0.self_attn.rotary_emb.inv_freq") is None and m.map_name("lm_head.weight") == "lm_head.weight"
    assert m.map_name("model.layers.1.mlp.up_proj.weight") == "layers.1.mlp.up_proj.weight" and m.missing(loader.load_tensors()) == []
    bare = llm.LLaMA(cfg)
    assert set(m.expected_weights()) == {k for k, _ in bare.named_parameters()}                # exactly the decoder's parameters
    assert len(m.expected_weights()) == 2 + 9 * cfg.num_hidden_layers and set(mapped) - set(m.expected_weights()) == {"lm_head.weight"}
    part = {k: v for k, v in loader.load_tensors().items() if "q_proj" not in k}
    assert m.missing(part) == [f"layers.{i}.self_attn.q_proj.weight" for i in range(cfg.num_hidden_layers)]
    assert llm.MistralWeightMapper(3).expected_weights() == llm.LLaMAWeightMapper(3).expected_weights()
    info = loader.tensor_info("model.norm.weight")
    assert isinstance(info, llm.TensorInfo) and info.dtype == "BF16" and info.shape == [cfg.hidden_size] and info.numel() == cfg.hidden_size
    assert loader.tensor_info("absent") is None
    pcfg = llm.PhiConfig(vocab_size=50, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4,
                         max_position_embeddings=32)
    phi = llm.PhiForCausalLM(pcfg)
    names = {k for k, _ in phi.named_parameters()}
    pm = llm.PhiWeightMapper(2)
    assert set(pm.expected_weights()) <= names and "layers.1.mlp.fc2.weight" in names and isinstance(phi.layers[0].mlp, llm.PhiMLP)
    assert pm.map_name("transformer.layers.0.mlp.fc1.bias") == "layers.0.mlp.fc1.bias" and pm.map_name("model.final_layernorm.bias") == "final_layernorm.bias"
    hf = {"model." + k if not k.startswith("lm_head") else k: v.detach() for k, v in phi.named_parameters()}
    fresh = llm.PhiForCausalLM(pcfg)
    res = llm.load_with_mapping(fresh, hf, "phi", strict=True)
    assert res.loaded_count == len(names)
    ids = torch.randint(0, 50, (1, 6))
    with torch.no_grad():
        assert torch.allclose(fresh.eval()(ids), phi.eval()(ids), atol=1e-5)
    assert llm.MistralAttention is llm.LLaMAAttention and llm.MistralMLP is llm.LLaMAMLP and llm.MistralDecoderLayer is llm.LLaMADecoderLayer
    with pytest.raises(NotImplementedError):
        llm.WeightMapper(1).map_name("x")


def test_text_generator_steps():
    cfg = llm.GenerationConfig.greedy(10).with_max_tokens(7).with_eos_token(2).with_eos_token(9).with_repetition_penalty(2.0)
    assert (cfg.max_new_tokens, cfg.eos_token_ids, cfg.repetition_penalty, cfg.do_sample) == (7, [2, 9], 2.0, False)
    g = llm.TextGenerator(cfg)
    lg = torch.tensor([2.0, -1.0, 4.0, 0.5])
    out = g.apply_repetition_penalty(lg, [0, 1])
    assert out.tolist() == [1.0, -2.0, 4.0, 0.5] and lg.tolist() == [2.0, -1.0, 4.0, 0.5]                # the input is left alone
    assert g.apply_repetition_penalty(lg, []).tolist() == lg.tolist() and g.apply_repetition_penalty(lg, None) is lg
    assert g.should_stop(9) and not g.should_stop(3) and int(g.argmax(lg)) == 2
    assert g.get_next_token([1.0, 5.0, 4.0], [1]) == 2                                                  # 5 / 2 < 4
    t = llm.TextGenerator(llm.GenerationConfig(temperature=0.5, top_k=2, top_p=None))
    assert t.apply_temperature(lg).tolist() == [4.0, -2.0, 8.0, 1.0]
    assert t.apply_top_k(lg).tolist() == [2.0, float("-inf"), 4.0, float("-inf")]
    batch = torch.stack([lg, lg.flip(0)])
    assert t.apply_top_k(batch).isinf().sum().item() == 4
    probs = torch.tensor([0.5, 0.3, 0.15, 0.05])
    p = llm.TextGenerator(llm.GenerationConfig(top_p=0.7))
    kept = p.apply_top_p(torch.log(probs))
    assert kept[:2].tolist() == pytest.approx(torch.log(probs[:2]).tolist()) and kept[2:].isinf().all()  # 0.5 + 0.3 reaches 0.7
    assert not llm.TextGenerator(llm.GenerationConfig(top_p=0.81)).apply_top_p(torch.log(probs))[2].isinf()
    full = t.process_logits(lg.unsqueeze(0))
    assert full.shape == (1, 4) and full[0].tolist() == [4.0, float("-inf"), 8.0, float("-inf")]
    torch.manual_seed(0)
    s = llm.TextGenerator(llm.GenerationConfig(top_k=1))
    assert {s.get_next_token([0.1, 3.0, 0.2]) for _ in range(5)} == {1}                                   # sampling from one candidate


def test_model_api_methods(tmp_path):
    torch.manual_seed(0)
    cfg, ref = _tiny_llama_dir(str(tmp_path / "ck"), dtype=torch.float32)
    model = llm.LLaMAForCausalLM.from_pretrained(str(tmp_path / "ck"), strict=True)
    assert model.config() == cfg and not model.training
    ids = torch.randint(0, cfg.vocab_size, (1, 10))
    with torch.no_grad():
        full = model(ids)
        assert torch.allclose(full, ref.eval()(ids), atol=1e-5)
        assert torch.equal(model.forward_ids(ids[0].float()), full)                          # 1-D float ids, as the reference passes them
        cache = model.create_kv_cache(1, 16)
        a = model.forward_with_cache(ids[:, :6], cache)
        b = model.forward_with_cache(ids[:, 6:], cache)                                      # positions continue from the cache
        assert cache.seq_len() == 10 and torch.allclose(torch.cat([a, b], 1), full, atol=1e-4)
        out = model.generate_greedy(ids[:, :4], max_new_tokens=5)
        nocache = ids[:, :4]
        for _ in range(5):
            nocache = torch.cat([nocache, model(nocache)[:, -1].argmax(-1, keepdim=True)], 1)
        assert torch.equal(out, nocache)
        bare = llm.LLaMA.from_pretrained(str(tmp_path / "ck"))
        assert isinstance(bare, llm.LLaMA) and torch.allclose(bare.forward_ids(ids), model.model(ids), atol=1e-6)
        layer = model.model.layers[0]
        x = torch.randn(1, 5, cfg.hidden_size)
        lc = llm.KVCache(1, 8, cfg.num_key_value_heads, cfg.head_dim())
        whole = layer.forward_with_cache(x, None)
        step = torch.cat([layer.forward_with_cache(x[:, :3], lc), layer.forward_with_cache(x[:, 3:], lc)], 1)
        assert torch.allclose(whole, step, atol=1e-5) and lc.seq_len == 5
        ac = llm.KVCache(1, 8, cfg.num_key_value_heads, cfg.head_dim())
        att = layer.self_attn
        assert torch.allclose(torch.cat([att.forward_with_cache(x[:, :2], ac), att.forward_with_cache(x[:, 2:], ac)], 1), att(x), atol=1e-5)
    w = {"pre.weight": torch.full((cfg.hidden_size,), 3.0), "other": torch.zeros(1)}
    assert layer.input_layernorm.load_weights(w, "pre.") == 1 and torch.all(layer.input_layernorm.weight == 3.0)
    layer.input_layernorm.load_weight(torch.ones(cfg.hidden_size))
    assert torch.all(layer.input_layernorm.weight == 1.0)
    with pytest.raises(ValueError):
        layer.input_layernorm.load_weight(torch.ones(3))
    src = {f"layers.1.{k}": v.detach().clone() for k, v in model.model.layers[1].named_parameters()}
    assert layer.load_weights(src, "layers.1.") == 9 and torch.equal(layer.mlp.up_proj.weight, model.model.layers[1].mlp.up_proj.weight)
    with pytest.raises(ValueError, match="layers.1.mlp.up_proj.weight"):
        layer.load_weights({"layers.1.mlp.up_proj.weight": torch.zeros(2, 2)}, "layers.1.")
    m = llm.MistralConfig.mistral_7b_instruct()
    assert m.sliding_window is None and m.rope_theta == 1e6 and llm.PhiConfig.phi2().rotary_dim() == 32 and llm.PhiConfig.phi1().rotary_dim() == 32
    pc = llm.PhiConfig.tiny()
    assert not llm.PhiForCausalLM.with_parallel_attn(pc, False).layers[0].parallel and llm.PhiForCausalLM.with_parallel_attn(pc).layers[0].parallel
    phi = llm.PhiForCausalLM(pc).eval()
    pids = torch.randint(0, pc.vocab_size, (1, 8))
    with torch.no_grad():
        cache = phi.create_kv_cache(1, 16)
        stepwise = torch.cat([phi.forward_with_cache(pids[:, :5], cache), phi.forward_with_cache(pids[:, 5:], cache)], 1)
        assert torch.allclose(stepwise, phi.forward_ids(pids), atol=1e-4)


def test_gpt2_and_bert_api_methods():
    torch.manual_seed(0)
    tiny = llm.GPT2LMHead.tiny().eval()
    assert tiny.config() == llm.GPT2Config.tiny() and isinstance(llm.GPT2.tiny(), llm.GPT2) and callable(llm.GPT2.small) and callable(llm.GPT2LMHead.xl)
    ids = torch.randint(0, tiny.cfg.vocab_size, (1, 9))
    with torch.no_grad():
        full = tiny(ids)
        h1, past = tiny.transformer.forward_with_past(ids[:, :4])
        h2, past = tiny.transformer.forward_with_past(ids[:, 4:], past)
        assert past.seq_len() == 9 and torch.allclose(torch.cat([h1, h2], 1), tiny.transformer(ids), atol=1e-4)
        cache = tiny.create_kv_cache(1, 16)
        stepwise = torch.cat([tiny.forward_with_cache(ids[:, :5], cache), tiny.forward_with_cache(ids[:, 5:], cache)], 1)
        assert torch.allclose(stepwise, full, atol=1e-4)
        greedy = tiny.generate_greedy(ids[:, :3], 4)
        ref = ids[:, :3]
        for _ in range(4):
            ref = torch.cat([ref, tiny(ref)[:, -1].argmax(-1, keepdim=True)], 1)
        assert torch.equal(greedy, ref)
        emb = tiny.transformer.wte
        assert torch.equal(emb.forward_ids(ids[0].float()), emb(ids))
        att = tiny.transformer.blocks[0].attention
        x = torch.randn(1, 6, tiny.cfg.n_embd)
        kc = llm.KVCache(1, 8, tiny.cfg.n_head, tiny.cfg.head_dim())
        parts = torch.cat([att.forward_with_cache(x[:, :4], kc), att.forward_with_cache(x[:, 4:], kc)], 1)
        assert torch.allclose(parts, att.forward_causal(x), atol=1e-5)
        m = att.create_causal_mask(4)
        assert m.shape == (4, 4) and torch.all(m.tril() == 0) and torch.isinf(m[0, 1]) and m[0, 1] < 0
    cfg = llm.BertConfig(vocab_size=40, hidden_size=16, num_hidden_layers=1, num_attention_heads=2, intermediate_size=32,
                         max_position_embeddings=12, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    bert = llm.Bert(cfg).eval()
    bids = torch.randint(0, 40, (2, 5))
    with torch.no_grad():
        seq, pooled = bert.forward_with_pooling(bids)
        assert seq.shape == (2, 5, 16) and pooled.shape == (2, 16) and torch.equal(bert.forward_ids(bids.float()), seq)
        nop = llm.Bert.with_pooler(cfg, False)
        assert nop.pooler is None and nop(bids)[1] is None and not any("pooler" in k for k, _ in nop.named_parameters())
        with pytest.raises(ValueError):
            nop.forward_with_pooling(bids)
        clf = llm.BertForSequenceClassification(cfg, 3).eval()
        assert torch.equal(clf.forward_classification(bids), clf(bids)) and clf(bids).shape == (2, 3)
        mlm = llm.BertForMaskedLM(cfg).eval()
        assert torch.equal(mlm.forward_mlm(bids), mlm(bids)) and mlm.config() is cfg


def test_loader_reports_and_embedding_lookup(tmp_path, capsys):
    cfg, _ = _tiny_llama_dir(str(tmp_path / "ck"), dtype=torch.float16)
    loader = llm.HFLoader.from_local(str(tmp_path / "ck"))
    assert loader.cache_dir() == str(tmp_path / "ck") and loader.tensors == {}
    loader.load_tensors()
    assert len(loader.tensors) == 22
    loader.print_tensor_info(limit=2)
    out = capsys.readouterr().out.splitlines()
    assert len(out) == 3 and "F16" in out[0] and out[2].startswith("22 tensors, ")
    from axonml_b200 import nn
    e = nn.Embedding(10, 4)
    assert torch.equal(e.lookup(torch.tensor([[1.0, 2.0]])), e(torch.tensor([[1, 2]])))
    with pytest.raises(IndexError):
        e.lookup(torch.tensor([10]))
    cell = nn.GRUCell(3, 5)
    h = torch.zeros(2, 5)
    assert torch.equal(cell.forward_step(torch.ones(2, 3), h), cell(torch.ones(2, 3), h))
    with pytest.raises(ValueError, match="expected input size 3, got 4"):
        cell.forward_step(torch.ones(2, 4), h)
    lc = nn.LSTMCell(3, 5)
    hh, cc = lc.forward_step(torch.ones(2, 3), (h, h))
    assert hh.shape == cc.shape == (2, 5)
    seq = nn.Sequential(nn.Linear(2, 2), nn.ReLU())
    ml = nn.ModuleList([nn.Linear(2, 2)])
    assert seq.len() == 2 and ml.len() == 1 and list(ml.iter_mut())[0] is ml[0]
