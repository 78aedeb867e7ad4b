"""Audio front end: container decoding, resampling and the log-mel features speech models take
(reference: src/audio/preprocessing*.rs, whisper_mel.rs, wav_writer.rs)."""
from .features import LogMel, mel_filter_bank
from .wav import decode_audio, read_wav, resample, write_wav

__all__ = ["LogMel", "mel_filter_bank", "decode_audio", "read_wav", "resample", "write_wav"]
