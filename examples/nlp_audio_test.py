"""Tour of the text and audio packages (the reference's crates/axonml/examples/nlp_audio_test.rs):
tokenizers, vocabulary, BPE training, a sentiment dataset, resampling, mel spectrogram, MFCC,
normalisation, noise, and a synthetic command dataset.

    python examples/nlp_audio_test.py
"""
import math

import torch

from axonml_b200 import audio, text


def main() -> dict:
    out = {}
    print("--- text ---")
    sentence = "Hello, world! This is Axonml ML framework."
    ws = text.WhitespaceTokenizer()
    print("whitespace:", ws.tokenize(sentence))
    print("character :", text.CharTokenizer().tokenize("Hello"))
    vocab = text.Vocab.from_text("the quick brown fox jumps over the lazy dog", 1)
    print("vocabulary size:", vocab.len(), " 'the' ->", vocab.token_to_index("the"), " 'quick' ->", vocab.token_to_index("quick"))
    enc = vocab.encode(ws.tokenize("the quick fox"))
    print("'the quick fox' ->", enc, "->", vocab.decode(enc))
    out["encoded"] = enc
    bpe = text.BasicBPETokenizer()
    bpe.train("low lower lowest newer newest", 10)
    out["bpe"] = bpe.tokenize("lower")
    print("BPE 'lower' ->", out["bpe"])
    ds = text.SyntheticSentimentDataset(100, 32, 1000)
    x, y = ds.get(0)
    print("sentiment sample:", tuple(x.shape), "label", y.tolist() if hasattr(y, "tolist") else y)
    print("\n--- audio ---")
    sr, dur, f0 = 16000, 0.5, 440.0
    n = int(sr * dur)
    wave = torch.sin(2 * math.pi * f0 * torch.arange(n) / sr)
    res = audio.Resample(16000, 8000).apply(wave)
    print(f"resample: {n} -> {res.shape[0]} samples")
    mel = audio.MelSpectrogram(sr, 400, 160, 40).apply(wave)
    mfcc = audio.MFCC(sr, 13, 40).apply(wave)
    print("mel spectrogram:", tuple(mel.shape), " MFCC:", tuple(mfcc.shape))
    norm = audio.NormalizeAudio().apply(wave * 0.3)
    noisy = audio.AddNoise(20.0).apply(wave)
    snr = 10 * torch.log10(wave.pow(2).mean() / (noisy - wave).pow(2).mean())
    print(f"normalised peak {float(norm.abs().max()):.3f}; noise at {float(snr):.1f} dB SNR")
    cmd = audio.SyntheticCommandDataset(10, 5)
    a, lab = cmd.get(3)
    print("command sample:", tuple(a.shape), "label", int(lab) if not hasattr(lab, "shape") or lab.dim() == 0 else lab.tolist())
    out.update({"resampled": res.shape[0], "mel": tuple(mel.shape), "mfcc": tuple(mfcc.shape), "snr_db": float(snr),
                "peak": float(norm.abs().max())})
    return out


if __name__ == "__main__":
    main()
