"""Unit tests of the text, audio and vision libraries on the CPU, one behaviour per test (the topics
of the reference's in-module and integration tests under crates/axonml-text, crates/axonml-audio and
crates/axonml-vision)."""
import math

import pytest
import torch

from axonml_b200 import audio as AU, data as D, nn, optim, text as TX, vision as V


# ------------------------------------------------------------------------------------- tokenizers
def test_whitespace_tokenizer_plain_and_lowercase():
    assert TX.WhitespaceTokenizer().tokenize("Hello  World\tfoo") == ["Hello", "World", "foo"]
    assert TX.WhitespaceTokenizer.lowercase().tokenize("Hello World") == ["hello", "world"]
    assert TX.WhitespaceTokenizer().tokenize("") == [] and TX.WhitespaceTokenizer().tokenize("   ") == []


def test_char_tokenizer_with_and_without_whitespace():
    assert TX.CharTokenizer().tokenize("a b") == ["a", " ", "b"]
    assert TX.CharTokenizer.no_whitespace().tokenize("a b\tc") == ["a", "b", "c"]


def test_word_punct_tokenizer_splits_punctuation():
    assert TX.WordPunctTokenizer().tokenize("Hello, world!") == ["Hello", ",", "world", "!"]
    assert TX.WordPunctTokenizer.lowercase().tokenize("It's OK.") == ["it", "'", "s", "ok", "."]


def test_ngram_tokenizers():
    assert TX.NGramTokenizer.word_ngrams(2).tokenize("a b c") == ["a b", "b c"]
    assert TX.NGramTokenizer.char_ngrams(3).tokenize("abcd") == ["abc", "bcd"]
    assert TX.NGramTokenizer.word_ngrams(3).tokenize("a b") in ([], ["a b"])


def test_bpe_training_merges_frequent_pairs_and_applies_them():
    bpe = TX.BasicBPETokenizer.new()
    bpe.train("low low low lower lowest low", 10)
    vocab = bpe.get_vocab()
    assert any(len(t.replace("</w>", "")) > 1 for t in vocab)
    toks = bpe.tokenize("low lower")
    assert "".join(toks).replace("</w>", "").replace(" ", "") == "lowlower" and len(toks) < len("lowlower")


def test_unigram_tokenizer_prefers_known_pieces():
    u = TX.UnigramTokenizer.from_tokens(["hello", "world", "hel", "lo"])
    assert "hello" in u.tokenize("hello") and isinstance(u.tokenize("unknownword"), list)


# ------------------------------------------------------------------------------------- vocabulary
def test_vocab_add_lookup_and_contains():
    v = TX.Vocab.new()
    assert v.is_empty() and v.add_token("cat") == 0 and v.add_token("dog") == 1 and v.add_token("cat") == 0
    assert v.len() == 2 and v.contains("dog") and not v.contains("fish")
    assert v.token_to_index("dog") == 1 and v.index_to_token(0) == "cat" and v.index_to_token(9) is None


def test_vocab_special_tokens_and_unknown():
    v = TX.Vocab.with_special_tokens()
    assert v.tokens()[:5] == ["<pad>", "<unk>", "<bos>", "<eos>", "<mask>"]
    assert v.pad_index() == 0 and v.unk_index_() == 1 and v.bos_index() == 2 and v.eos_index() == 3
    v.add_token("known")
    assert v.encode(["known", "never-seen"]) == [5, 1]
    assert TX.Vocab.new().token_to_index("x") is None


def test_vocab_encode_decode_round_trip():
    v = TX.Vocab.from_tokens(["b", "a", "b", "c", "b", "a"])
    ids = v.encode(["a", "b", "c"])
    assert v.decode(ids) == ["a", "b", "c"] and v.token_to_index("b") < v.token_to_index("a") < v.token_to_index("c")
    assert v.encode_tensor(["a", "b"]).dtype == torch.long


def test_vocab_from_text_with_minimum_frequency():
    v = TX.Vocab.from_text("the cat the dog the end", 2)
    assert v.contains("the") and not v.contains("cat")
    assert TX.Vocab.from_text("a b", TX.WhitespaceTokenizer().tokenize, 1).contains("b")


# ---------------------------------------------------------------------------------- text datasets
def test_text_dataset_pads_and_truncates():
    tok = TX.WhitespaceTokenizer()
    ds = TX.TextDataset.from_samples([("good movie", 1), ("bad bad bad film really", 0)], tok.tokenize, 1, 4)
    assert ds.len() == 2 and ds.num_classes() == 2 and ds.max_length() == 4
    x0, y0 = ds.get(0)
    x1, _ = ds.get(1)
    assert x0.shape == (4,) and x1.shape == (4,) and int(y0) == 1
    assert x0[2:].tolist() == [0, 0] and 0 not in x1.tolist()


def test_language_model_dataset_targets_are_shifted_inputs():
    ds = TX.LanguageModelDataset(list(range(20)), 5)
    x, y = ds.get(2)
    assert x.shape == (5,) and y.tolist() == (x + 1).tolist() and ds.len() >= 3
    v = TX.Vocab.from_text("a b c d e f g h", 1)
    lm = TX.LanguageModelDataset.from_text("a b c d e f g h", v, TX.WhitespaceTokenizer().tokenize, 3)
    assert lm.len() > 0 and lm.vocab() is v


def test_synthetic_sentiment_is_deterministic_and_learnable_shape():
    a, b = TX.SyntheticSentimentDataset(50, 16, 100, seed=1), TX.SyntheticSentimentDataset(50, 16, 100, seed=1)
    assert a.len() == 50 and a.get(7)[0].equal(b.get(7)[0]) and int(a.get(7)[1]) == int(b.get(7)[1])
    labels = {int(a.get(i)[1]) for i in range(50)}
    assert labels == {0, 1} and a.get(0)[0].shape == (16,) and int(a.get(0)[0].max()) < 100
    assert TX.SyntheticSentimentDataset.small().len() > 0


def test_synthetic_seq2seq_tasks():
    r = TX.SyntheticSeq2SeqDataset.reverse_task(10, 6, 20)
    src, tgt = r.get(0)
    assert tgt.tolist() == src.flip(0).tolist()
    c = TX.SyntheticSeq2SeqDataset.copy_task(10, 6, 20)
    src, tgt = c.get(3)
    assert tgt.equal(src)


def test_text_dataset_feeds_a_dataloader():
    ds = TX.SyntheticSentimentDataset(32, 8, 50)
    batches = list(D.DataLoader(ds, 8))
    assert len(batches) == 4 and batches[0].data.shape == (8, 8) and batches[0].targets.shape[0] == 8


# ------------------------------------------------------------------------------- audio transforms
def _tone(freq=440.0, sr=16000, dur=0.5):
    t = torch.arange(int(sr * dur)) / sr
    return torch.sin(2 * math.pi * freq * t)


def test_resample_changes_length_and_keeps_pitch():
    x = _tone(440.0, 16000)
    y = AU.Resample(16000, 8000).apply(x)
    assert abs(y.numel() - x.numel() // 2) <= 1
    spec = torch.fft.rfft(y).abs()
    assert abs(int(spec.argmax()) * 8000 / y.numel() - 440.0) < 10
    assert AU.Resample(16000, 16000).apply(x).equal(x)


def test_mel_spectrogram_and_mfcc_shapes_and_peak_band():
    low, high = AU.MelSpectrogram().apply(_tone(300.0)), AU.MelSpectrogram().apply(_tone(3000.0))
    assert low.shape[0] == 40 and low.shape == high.shape and torch.isfinite(low).all()
    assert int(low.mean(1).argmax()) < int(high.mean(1).argmax())
    m = AU.MFCC(16000, 13, 40).apply(_tone())
    assert m.shape[0] == 13 and torch.isfinite(m).all()
    assert AU.MelSpectrogram.with_params(8000, 256, 64, 20).apply(_tone(sr=8000)).shape[0] == 20


def test_mel_filterbank_rows_are_triangles_over_increasing_centres():
    fb = AU.mel_filterbank(10, 256, 16000)
    assert fb.shape == (10, 129) and float(fb.min()) >= 0 and float(fb.max()) <= 1.0 + 1e-6
    centres = fb.argmax(1).tolist()
    assert centres == sorted(centres) and len(set(centres)) == 10


def test_time_stretch_and_pitch_shift():
    x = _tone()
    assert abs(AU.TimeStretch(2.0).apply(x).numel() - x.numel() // 2) <= 2
    assert abs(AU.TimeStretch(0.5).apply(x).numel() - x.numel() * 2) <= 2
    y = AU.PitchShift(12.0).apply(x)
    assert y.numel() == x.numel()
    f = int(torch.fft.rfft(y).abs().argmax()) * 16000 / y.numel()
    assert abs(f - 880.0) < 10                                       # one octave up from 440 Hz
    down = AU.PitchShift(-12.0).apply(x)
    assert abs(int(torch.fft.rfft(down).abs().argmax()) * 16000 / down.numel() - 220.0) < 10
    assert float(y.pow(2).mean().sqrt()) == pytest.approx(float(x.pow(2).mean().sqrt()), rel=1e-3)
    assert AU.PitchShift(0.0).apply(x).equal(x) and AU.PitchShift(3.0).apply(torch.randn(2, 1600)).shape == (2, 1600)


def test_add_noise_reaches_the_requested_snr():
    torch.manual_seed(0)
    x = _tone()
    y = AU.AddNoise(10.0).apply(x)
    snr = 10 * math.log10(float(x.pow(2).mean()) / float((y - x).pow(2).mean()))
    assert abs(snr - 10.0) < 1.0


def test_normalize_and_trim_silence():
    x = 0.25 * _tone()
    assert float(AU.NormalizeAudio().apply(x).abs().max()) == pytest.approx(1.0, abs=1e-5)
    assert float(AU.NormalizeAudio(0.5).apply(x).abs().max()) == pytest.approx(0.5, abs=1e-5)
    padded = torch.cat([torch.zeros(1000), _tone(dur=0.1), torch.zeros(2000)])
    t = AU.TrimSilence(-40.0).apply(padded)
    assert 1500 <= t.numel() <= 1700 and float(t[:10].abs().max()) > 0


# --------------------------------------------------------------------------------- audio datasets
def test_synthetic_command_dataset_classes_are_distinguishable():
    ds = AU.SyntheticCommandDataset(40, 4, 8000, 0.25)
    assert ds.len() == 40 and ds.num_classes() == 4 and ds.sample_rate() == 8000
    x, y = ds.get(0)
    assert x.shape == (2000,) and float(x.abs().max()) <= 1.5 and 0 <= int(y) < 4
    peaks = {}
    for i in range(40):
        w, l = ds.get(i)
        peaks.setdefault(int(l), []).append(int(torch.fft.rfft(w).abs().argmax()))
    means = sorted(sum(v) / len(v) for v in peaks.values())
    assert len(peaks) == 4 and all(b - a > 1 for a, b in zip(means, means[1:]))
    with pytest.raises(IndexError):
        ds.get(40)
    assert len(list(ds)) == 40 and ds[-1][0].equal(ds.get(39)[0])


def test_music_and_speaker_datasets():
    m = AU.SyntheticMusicDataset(10, 3, 8000, 0.25)
    assert m.len() == 10 and m.num_genres() == 3 and m.get(0)[0].shape == (2000,)
    s = AU.SyntheticSpeakerDataset(10, 4, 8000, 0.25)
    assert s.num_speakers() == 4 and {int(s.get(i)[1]) for i in range(10)} <= set(range(4))


def test_audio_classification_and_seq2seq_datasets():
    waves = [torch.randn(100) for _ in range(6)]
    ds = AU.AudioClassificationDataset(waves, [0, 1, 2, 0, 1, 2], 8000, 3, one_hot=True)
    x, y = ds.get(4)
    assert x.equal(waves[4]) and y.tolist() == [0.0, 1.0, 0.0] and ds.num_classes() == 3
    s2s = AU.AudioSeq2SeqDataset.noise_reduction_task(5, 200, 0.1) if hasattr(AU.AudioSeq2SeqDataset, "noise_reduction_task") else None
    src, tgt = s2s.get(0)
    assert src.shape == tgt.shape and not src.equal(tgt)


def test_audio_pipeline_through_a_dataloader():
    ds = AU.SyntheticCommandDataset(16, 4, 8000, 0.25)
    mel = AU.MelSpectrogram.with_params(8000, 256, 128, 20)
    feats = D.MapDataset(ds, lambda x, y: (mel.apply(x), y))
    b = next(iter(D.DataLoader(feats, 4)))
    assert b.data.shape[:2] == (4, 20) and b.targets.shape == (4,)


# ------------------------------------------------------------------------------- vision datasets
def test_synthetic_mnist_is_deterministic_and_in_range():
    a, b = V.SyntheticMNIST(20, seed=3), V.SyntheticMNIST(20, seed=3)
    x, y = a.get(5)
    assert x.shape == (1, 28, 28) and 0.0 <= float(x.min()) and float(x.max()) <= 1.0 and 0 <= int(y) < 10
    assert x.equal(b.get(5)[0]) and a.len() == 20 and a.num_classes() == 10
    with pytest.raises(IndexError):
        a.get(20)
    assert sum(1 for _ in a) == 20


def test_synthetic_cifar_variants():
    c10 = V.SyntheticCIFAR.cifar10(30)
    x, y = c10.get(0)
    assert x.shape == (3, 32, 32) and 0 <= int(y) < 10 and len(c10.class_names()) == 10 and "airplane" in c10.class_names()
    c100 = V.SyntheticCIFAR.cifar100(300)
    assert c100.num_classes() == 100 and len({int(c100.get(i)[1]) for i in range(300)}) > 50
    assert not c10.get(0)[0].equal(c10.get(1)[0])


# --------------------------------------------------------------------------------- vision models
def test_lenet_parameter_count_and_forward():
    m = V.LeNet.new()
    assert m.num_parameters() == 61706 or m.num_parameters() == 44426            # 32x32 / 28x28 inputs
    assert m(torch.randn(2, 1, 28, 28)).shape == (2, 10)
    assert V.LeNet.for_cifar10()(torch.randn(2, 3, 32, 32)).shape == (2, 10)


def test_mlp_flattens_images_and_simple_cnn_runs():
    assert V.MLP.for_mnist()(torch.randn(3, 1, 28, 28)).shape == (3, 10)
    assert V.MLP(12, [8, 4], 3)(torch.randn(5, 12)).shape == (5, 3)
    c = V.SimpleCNN.for_mnist()
    assert c(torch.randn(2, 1, 28, 28)).shape == (2, 10) and c.num_classes() == 10 and c.input_channels() == 1
    assert V.SimpleCNN.for_cifar10()(torch.randn(2, 3, 32, 32)).shape == (2, 10)


def test_resnet_blocks_and_small_forward():
    blk = V.BasicBlock(16, 16)
    x = torch.randn(2, 16, 8, 8)
    assert blk(x).shape == x.shape and V.BasicBlock.expansion == 1 and V.Bottleneck.expansion == 4
    assert V.BasicBlock(16, 32, stride=2)(x).shape == (2, 32, 4, 4)
    m = V.resnet18(10).eval()
    assert m(torch.randn(1, 3, 64, 64)).shape == (1, 10)
    assert 11_000_000 < m.num_parameters() < 11_400_000


def test_vgg_creation_and_modes():
    m = V.vgg11(10)
    assert sum(1 for l in m.modules() if isinstance(l, nn.Conv2d)) == 8
    bn = V.vgg11_bn(10)
    assert sum(1 for l in bn.modules() if isinstance(l, nn.BatchNorm2d)) == 8
    assert sum(1 for l in V.vgg16(10).modules() if isinstance(l, nn.Conv2d)) == 13
    assert not m.eval().is_training() and m.train().is_training()


def test_vision_transformer_and_encoder_shapes():
    vit = V.VisionTransformer(32, 8, 3, 5, 32, 2, 4).eval()
    assert vit(torch.randn(2, 3, 32, 32)).shape == (2, 5)
    pe = V.PositionalEncoding(16, 50)
    z = torch.zeros(1, 10, 16)
    out = pe(z)
    assert out.shape == (1, 10, 16) and out[0, 0, 0].item() == 0.0 and out[0, 0, 1].item() == 1.0
    with pytest.raises(ValueError):
        pe(torch.zeros(1, 51, 16))


# ------------------------------------------------------------------------------------ vision hub
def test_model_registry_and_info():
    reg = V.model_registry()
    assert "resnet18" in reg and reg["resnet18"].num_classes == 1000 and reg["resnet18"].size_bytes > 10 ** 7
    assert V.model_info("resnet18").name == "resnet18" and V.model_info("no-such") is None
    assert len(V.list_models()) == len(reg) and all(m.url.startswith("http") for m in V.list_models())


def test_cache_paths_follow_the_cache_root(tmp_path, monkeypatch):
    monkeypatch.setenv("AXONML_HUB_CACHE", str(tmp_path))
    assert V.cache_dir().startswith(str(tmp_path)) and V.cached_path("resnet18").endswith("resnet18.safetensors")
    assert not V.is_cached("resnet18")


def test_hub_state_dict_round_trip(tmp_path):
    sd = {"fc.weight": torch.randn(3, 4), "fc.bias": torch.zeros(3)}
    path = str(tmp_path / "w.bin")
    V.save_state_dict(sd, path)
    back = V.load_state_dict(path)
    assert set(back) == set(sd) and torch.allclose(back["fc.weight"], sd["fc.weight"])


# -------------------------------------------------------------------------------- vision transforms
def test_resize_and_center_crop():
    img = torch.rand(3, 20, 30)
    assert V.Resize.new(10, 15).apply(img).shape == (3, 10, 15) and V.Resize.square(8).apply(img).shape == (3, 8, 8)
    assert V.Resize(12).apply(torch.rand(2, 3, 20, 30)).shape == (2, 3, 12, 12)
    c = V.CenterCrop.square(10).apply(img)
    assert c.shape == (3, 10, 10) and c.equal(img[:, 5:15, 10:20])


def test_flips_rotation_and_grayscale():
    img = torch.arange(12.0).reshape(1, 3, 4)
    assert V.RandomHorizontalFlip.with_probability(1.0).apply(img).equal(img.flip(-1))
    assert V.RandomVerticalFlip.with_probability(1.0).apply(img).equal(img.flip(-2))
    assert V.RandomHorizontalFlip.with_probability(0.0).apply(img).equal(img)
    assert V.RandomRotation.with_angles([180]).apply(img).equal(img.flip(-1).flip(-2))
    assert V.RandomRotation.with_angles([90]).apply(img).shape == (1, 4, 3)
    rgb = torch.rand(3, 5, 5)
    g = V.Grayscale.new().apply(rgb)
    assert g.shape == (1, 5, 5) and torch.allclose(g[0], 0.299 * rgb[0] + 0.587 * rgb[1] + 0.114 * rgb[2], atol=1e-6)
    assert V.Grayscale.with_channels(3).apply(rgb).shape == (3, 5, 5)


def test_image_normalize_pad_to_tensor_and_jitter():
    x = torch.full((3, 2, 2), 0.5)
    n = V.ImageNormalize.imagenet().apply(x)
    assert n[:, 0, 0].tolist() == pytest.approx([(0.5 - 0.485) / 0.229, (0.5 - 0.456) / 0.224, (0.5 - 0.406) / 0.225])
    p = V.Pad.new(2).with_fill(1.0).apply(torch.zeros(1, 3, 3))
    assert p.shape == (1, 7, 7) and p[0, 0, 0].item() == 1.0 and p[0, 3, 3].item() == 0.0
    assert V.Pad.asymmetric(1, 2, 3, 4).apply(torch.zeros(1, 5, 5)).shape == (1, 12, 8)
    hwc = torch.randint(0, 256, (4, 6, 3), dtype=torch.uint8)
    t = V.ToTensorImage().apply(hwc)
    assert t.shape == (3, 4, 6) and float(t.max()) <= 1.0
    j = V.ColorJitter(0.4, 0.4, 0.4).apply(torch.rand(3, 8, 8))
    assert j.shape == (3, 8, 8) and 0.0 <= float(j.min()) and float(j.max()) <= 1.0


def test_lenet_learns_synthetic_mnist():
    torch.manual_seed(0)
    ds = V.SyntheticMNIST(256)
    model, opt, loss_fn = V.LeNet.new(), None, nn.CrossEntropyLoss()
    opt = optim.Adam(model.parameters(), lr=2e-3)
    first = last = None
    for _ in range(3):
        for b in D.DataLoader(ds, 32, shuffle=True):
            opt.zero_grad()
            loss = loss_fn(model(b.data), b.targets)
            loss.backward()
            opt.step()
            first = first if first is not None else loss.item()
            last = loss.item()
    assert last < first * 0.7
