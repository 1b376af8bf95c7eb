"""Audio processing (crates/axonml-audio)."""
from .datasets import (AudioClassificationDataset, AudioSeq2SeqDataset, SyntheticCommandDataset, SyntheticMusicDataset,
                       SyntheticSpeakerDataset)
from .transforms import (MFCC, AddNoise, MelSpectrogram, NormalizeAudio, PitchShift, Resample, TimeStretch,
                         TrimSilence, mel_filterbank)
