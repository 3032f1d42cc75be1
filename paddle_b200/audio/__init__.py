"""``paddle.audio`` (python/paddle/audio/): window functions, mel / dB helpers, spectrogram feature layers, wav IO."""
from __future__ import annotations

import math

import torch

from .._core.tensor import as_tensor
from ..nn.layer.layers import Layer


def _p(x):
    return x.as_subclass(torch.Tensor) if isinstance(x, torch.Tensor) else torch.as_tensor(x)


class functional:
    @staticmethod
    def get_window(window, win_length, fftbins=True, dtype="float64"):
        """Window by name, or ``(name, parameter...)`` for the parametrised ones (python/paddle/audio/functional/
        window.py ``get_window``): hamming, hann, gaussian (std), general_gaussian (power, width), exponential (tau),
        triang, bohman, blackman, cosine, tukey (alpha), taylor (nbar, sll), bartlett, kaiser (beta), nuttall;
        ``fftbins`` gives the periodic form used with an FFT."""
        from .._core import dtype as _dt
        args = ()
        if isinstance(window, (tuple, list)):
            window, args = window[0], tuple(window[1:])
        if not isinstance(window, str):
            raise ValueError(f"The window must be a str or a tuple of (str, parameters), got {type(window)}")
        if window in ("gaussian", "exponential", "kaiser") and not args:
            raise ValueError(f"The '{window}' window needs one or more parameters -- pass a tuple.")
        n = int(win_length)
        m = n + 1 if fftbins else n                      # periodic form: one extra point, last one dropped
        k = torch.arange(m, dtype=torch.float64)

        def cos_sum(coeffs):
            w = torch.zeros(m, dtype=torch.float64)
            for i, a in enumerate(coeffs):
                w = w + ((-1) ** i) * a * torch.cos(2 * math.pi * i * k / max(m - 1, 1))
            return w
        c = (m - 1) / 2.0
        if window in ("rect", "boxcar", "ones"):
            w = torch.ones(m, dtype=torch.float64)
        elif window == "hann":
            w = cos_sum([0.5, 0.5])
        elif window == "hamming":
            w = cos_sum([0.54, 0.46])
        elif window == "blackman":
            w = cos_sum([0.42, 0.5, 0.08])
        elif window == "nuttall":
            w = cos_sum([0.3635819, 0.4891775, 0.1365995, 0.0106411])
        elif window == "bartlett":
            w = 1.0 - torch.abs(2.0 * k / max(m - 1, 1) - 1.0)
        elif window == "triang":
            kk = torch.arange(1, (m + 1) // 2 + 1, dtype=torch.float64)
            half = (2 * kk - 1.0) / m if m % 2 == 0 else 2 * kk / (m + 1.0)
            w = torch.cat([half, half.flip(0)]) if m % 2 == 0 else torch.cat([half, half[:-1].flip(0)])
        elif window == "cosine":
            w = torch.sin(math.pi / m * (k + 0.5))
        elif window == "bohman":
            fac = torch.abs(torch.linspace(-1, 1, m, dtype=torch.float64)[1:-1])
            mid = (1 - fac) * torch.cos(math.pi * fac) + 1.0 / math.pi * torch.sin(math.pi * fac)
            w = torch.cat([torch.zeros(1, dtype=torch.float64), mid, torch.zeros(1, dtype=torch.float64)])
        elif window == "gaussian":
            w = torch.exp(-0.5 * ((k - c) / float(args[0])) ** 2)
        elif window == "general_gaussian":
            p_, sig = (float(args[0]), float(args[1])) if len(args) >= 2 else (1.0, float(args[0]) if args else 1.0)
            w = torch.exp(-0.5 * torch.abs((k - c) / sig) ** (2 * p_))
        elif window == "exponential":
            tau = float(args[0])
            w = torch.exp(-torch.abs(k - c) / tau)
        elif window == "kaiser":
            beta = float(args[0])
            w = torch.special.i0(beta * torch.sqrt((1 - ((k - c) / c) ** 2).clamp(min=0))) / torch.special.i0(torch.tensor(beta, dtype=torch.float64))
        elif window == "tukey":
            alpha = float(args[0]) if args else 0.5
            if alpha <= 0:
                w = torch.ones(m, dtype=torch.float64)
            elif alpha >= 1:
                w = cos_sum([0.5, 0.5])
            else:
                width = int(math.floor(alpha * (m - 1) / 2.0))
                n1, n3 = k[:width + 1], k[m - width - 1:]
                w1 = 0.5 * (1 + torch.cos(math.pi * (-1 + 2.0 * n1 / alpha / (m - 1))))
                w3 = 0.5 * (1 + torch.cos(math.pi * (-2.0 / alpha + 1 + 2.0 * n3 / alpha / (m - 1))))
                w = torch.cat([w1, torch.ones(m - 2 * (width + 1), dtype=torch.float64), w3])
        elif window == "taylor":
            nbar, sll = (int(args[0]) if args else 4), (float(args[1]) if len(args) > 1 else 30.0)
            B = 10 ** (sll / 20)
            A = math.acosh(B) / math.pi
            s2 = nbar ** 2 / (A ** 2 + (nbar - 0.5) ** 2)
            ma = torch.arange(1, nbar, dtype=torch.float64)
            Fm = torch.empty(nbar - 1, dtype=torch.float64)
            signs = torch.ones(nbar - 1, dtype=torch.float64)
            signs[1::2] = -1
            m2 = ma * ma
            for mi in range(len(ma)):
                numer = signs[mi] * torch.prod(1 - m2[mi] / s2 / (A ** 2 + (ma - 0.5) ** 2))
                denom = 2 * torch.prod(1 - m2[mi] / m2[:mi]) * torch.prod(1 - m2[mi] / m2[mi + 1:])
                Fm[mi] = numer / denom
            def W(nn):
                return 1 + 2 * torch.matmul(Fm.unsqueeze(0), torch.cos(2 * math.pi * ma.unsqueeze(1) * (nn - m / 2.0 + 0.5) / m))
            w = W(k).reshape(-1)
            w = w / W(torch.tensor([(m - 1) / 2.0], dtype=torch.float64)).reshape(-1)
        else:
            raise ValueError(f"Unknown window type: {window}")
        w = w[:n] if fftbins else w
        return as_tensor(w.to(_dt.to_torch(dtype)))

    @staticmethod
    def hz_to_mel(freq, htk=False):
        f = torch.as_tensor(freq, dtype=torch.float64)
        if htk:
            out = 2595.0 * torch.log10(1.0 + f / 700.0)
        else:
            f_sp, min_log_hz = 200.0 / 3, 1000.0
            min_log_mel, logstep = min_log_hz / f_sp, math.log(6.4) / 27.0
            out = torch.where(f >= min_log_hz, min_log_mel + torch.log(f.clamp(min=1e-10) / min_log_hz) / logstep, f / f_sp)
        return float(out) if out.dim() == 0 and not isinstance(freq, torch.Tensor) else as_tensor(out)

    @staticmethod
    def mel_to_hz(mel, htk=False):
        m = torch.as_tensor(mel, dtype=torch.float64)
        if htk:
            out = 700.0 * (10.0 ** (m / 2595.0) - 1.0)
        else:
            f_sp, min_log_hz = 200.0 / 3, 1000.0
            min_log_mel, logstep = min_log_hz / f_sp, math.log(6.4) / 27.0
            out = torch.where(m >= min_log_mel, min_log_hz * torch.exp(logstep * (m - min_log_mel)), f_sp * m)
        return float(out) if out.dim() == 0 and not isinstance(mel, torch.Tensor) else as_tensor(out)

    @staticmethod
    def mel_frequencies(n_mels=64, f_min=0.0, f_max=11025.0, htk=False, dtype="float32"):
        lo, hi = functional.hz_to_mel(f_min, htk), functional.hz_to_mel(f_max, htk)
        return as_tensor(_p(functional.mel_to_hz(torch.linspace(lo, hi, n_mels, dtype=torch.float64), htk)).float())

    @staticmethod
    def fft_frequencies(sr, n_fft, dtype="float32"):
        return as_tensor(torch.linspace(0, sr / 2, 1 + n_fft // 2))

    @staticmethod
    def compute_fbank_matrix(sr, n_fft, n_mels=64, f_min=0.0, f_max=None, htk=False, norm="slaney", dtype="float32"):
        f_max = f_max or sr / 2
        fft_f = _p(functional.fft_frequencies(sr, n_fft)).double()
        mel_f = _p(functional.mel_to_hz(torch.linspace(functional.hz_to_mel(f_min, htk), functional.hz_to_mel(f_max, htk),
                                                       n_mels + 2, dtype=torch.float64), htk)).double()
        fdiff = mel_f[1:] - mel_f[:-1]
        ramps = mel_f[:, None] - fft_f[None]
        lower, upper = -ramps[:-2] / fdiff[:-1, None], ramps[2:] / fdiff[1:, None]
        w = torch.clamp(torch.minimum(lower, upper), min=0)
        if norm == "slaney":
            w = w * (2.0 / (mel_f[2:] - mel_f[:-2]))[:, None]
        return as_tensor(w.float())

    @staticmethod
    def power_to_db(spect, ref_value=1.0, amin=1e-10, top_db=80.0):
        s = _p(spect)
        db = 10.0 * torch.log10(s.clamp(min=amin)) - 10.0 * math.log10(max(amin, ref_value))
        if top_db is not None:
            db = torch.maximum(db, db.max() - top_db)
        return as_tensor(db)

    @staticmethod
    def create_dct(n_mfcc, n_mels, norm="ortho", dtype="float32"):
        n = torch.arange(n_mels, dtype=torch.float32)
        k = torch.arange(n_mfcc, dtype=torch.float32)[:, None]
        dct = torch.cos(math.pi / n_mels * (n + 0.5) * k)
        if norm == "ortho":
            dct[0] *= 1.0 / math.sqrt(2.0)
            dct *= math.sqrt(2.0 / n_mels)
        else:
            dct *= 2.0
        return as_tensor(dct.t().contiguous())


class features:
    class Spectrogram(Layer):
        def __init__(self, n_fft=512, hop_length=None, win_length=None, window="hann", power=2.0, center=True,
                     pad_mode="reflect", dtype="float32"):
            super().__init__()
            self.n_fft, self.hop, self.win_length = n_fft, hop_length or n_fft // 4, win_length or n_fft
            self.power, self.center, self.pad_mode = power, center, pad_mode
            self.window = _p(functional.get_window(window, self.win_length)).float()

        def forward(self, x):
            s = torch.stft(_p(x), self.n_fft, self.hop, self.win_length, self.window.to(x.device), self.center,
                           self.pad_mode, return_complex=True)
            return as_tensor(s.abs() ** self.power)

    class MelSpectrogram(Layer):
        def __init__(self, sr=22050, n_fft=512, hop_length=None, win_length=None, window="hann", power=2.0, center=True,
                     pad_mode="reflect", n_mels=64, f_min=50.0, f_max=None, htk=False, norm="slaney", dtype="float32"):
            super().__init__()
            self.spec = features.Spectrogram(n_fft, hop_length, win_length, window, power, center, pad_mode)
            self.fbank = _p(functional.compute_fbank_matrix(sr, n_fft, n_mels, f_min, f_max, htk, norm))

        def forward(self, x):
            return as_tensor(torch.matmul(self.fbank.to(x.device), _p(self.spec(x))))

    class LogMelSpectrogram(Layer):
        def __init__(self, sr=22050, n_fft=512, hop_length=None, win_length=None, window="hann", power=2.0, center=True,
                     pad_mode="reflect", n_mels=64, f_min=50.0, f_max=None, htk=False, norm="slaney", ref_value=1.0,
                     amin=1e-10, top_db=None, dtype="float32"):
            super().__init__()
            self.mel = features.MelSpectrogram(sr, n_fft, hop_length, win_length, window, power, center, pad_mode, n_mels,
                                               f_min, f_max, htk, norm)
            self.ref_value, self.amin, self.top_db = ref_value, amin, top_db

        def forward(self, x):
            return functional.power_to_db(self.mel(x), self.ref_value, self.amin, self.top_db)

    class MFCC(Layer):
        def __init__(self, sr=22050, n_mfcc=40, n_fft=512, hop_length=None, win_length=None, window="hann", power=2.0,
                     center=True, pad_mode="reflect", n_mels=64, f_min=50.0, f_max=None, htk=False, norm="slaney",
                     ref_value=1.0, amin=1e-10, top_db=None, dtype="float32"):
            super().__init__()
            self.logmel = features.LogMelSpectrogram(sr, n_fft, hop_length, win_length, window, power, center, pad_mode,
                                                     n_mels, f_min, f_max, htk, norm, ref_value, amin, top_db)
            self.dct = _p(functional.create_dct(n_mfcc, n_mels))

        def forward(self, x):
            lm = _p(self.logmel(x))
            return as_tensor(torch.matmul(lm.transpose(-1, -2), self.dct.to(lm.device)).transpose(-1, -2))


class backends:
    @staticmethod
    def list_available_backends():
        return ["wave_backend"]

    @staticmethod
    def get_current_backend():
        return "wave_backend"

    @staticmethod
    def set_backend(name):
        if name != "wave_backend":
            raise NotImplementedError("only the built-in wave backend is available")


def load(filepath, frame_offset=0, num_frames=-1, normalize=True, channels_first=True):
    import wave

    import numpy as np
    with wave.open(filepath, "rb") as f:
        sr, nch, width = f.getframerate(), f.getnchannels(), f.getsampwidth()
        f.setpos(frame_offset)
        raw = f.readframes(f.getnframes() - frame_offset if num_frames < 0 else num_frames)
    dt = {1: np.uint8, 2: np.int16, 4: np.int32}[width]
    a = np.frombuffer(raw, dtype=dt).reshape(-1, nch)
    t = torch.from_numpy(a.astype(np.float32))
    if normalize:
        t = (t - 128.0) / 128.0 if width == 1 else t / float(2 ** (8 * width - 1))
    return as_tensor(t.t().contiguous() if channels_first else t), sr


def save(filepath, src, sample_rate, channels_first=True, encoding=None, bits_per_sample=16):
    import wave

    import numpy as np
    t = _p(src).detach().cpu()
    t = t.t() if channels_first else t
    a = (t.clamp(-1, 1) * (2 ** (bits_per_sample - 1) - 1)).numpy().astype({16: np.int16, 32: np.int32}[bits_per_sample])
    with wave.open(filepath, "wb") as f:
        f.setnchannels(a.shape[1]), f.setsampwidth(bits_per_sample // 8), f.setframerate(sample_rate)
        f.writeframes(a.tobytes())


def info(filepath):
    import wave
    with wave.open(filepath, "rb") as f:
        class _Info:
            sample_rate, num_frames, num_channels, bits_per_sample = f.getframerate(), f.getnframes(), f.getnchannels(), 8 * f.getsampwidth()
            encoding = "PCM_S"
        return _Info


# ----------------------------------------------------------------------------- datasets + importable submodules
class _AudioFolderDataset:
    """Common part of the audio classification datasets (python/paddle/audio/datasets/dataset.py): a list of wave
    files with labels; items are ``(feature, label)`` with ``feat_type`` in raw / spectrogram / melspectrogram /
    logmelspectrogram / mfcc."""

    def __init__(self, files, labels, feat_type="raw", sample_rate=None, **kwargs):
        self.files, self.labels, self.feat_type, self.sample_rate, self.feat_config = files, labels, feat_type, sample_rate, kwargs
        table = {"spectrogram": features.Spectrogram, "melspectrogram": features.MelSpectrogram,
                 "logmelspectrogram": features.LogMelSpectrogram, "mfcc": features.MFCC}
        if feat_type != "raw" and feat_type not in table:
            raise RuntimeError(f"Unknown feat_type: {feat_type}, it must be one in {['raw', *table]}")
        self._extract = None if feat_type == "raw" else table[feat_type]

    def __len__(self):
        return len(self.files)

    def __getitem__(self, idx):
        wav, sr = load(self.files[idx])
        x = wav[0] if wav.dim() == 2 else wav
        if self._extract is not None:
            cfg = dict(self.feat_config)
            if self.feat_type != "spectrogram":
                cfg.setdefault("sr", sr)
            x = self._extract(**cfg)(x.reshape([1, -1]))[0]
        return x, self.labels[idx]


class _Datasets:
    class ESC50(_AudioFolderDataset):
        """ESC-50 environmental sounds: ``<root>/audio/*.wav`` and ``<root>/meta/esc50.csv``; ``split`` is the fold
        held out for the dev set.  The archive has to be present locally (``data_dir``): nothing is downloaded."""

        def __init__(self, mode="train", split=1, feat_type="raw", archive=None, data_dir=None, **kwargs):
            import csv
            import os
            root = data_dir or os.path.expanduser("~/.cache/paddle/dataset/ESC-50-master")
            meta = os.path.join(root, "meta", "esc50.csv")
            if not os.path.exists(meta):
                raise RuntimeError(f"ESC50 is not available offline: expected {meta}")
            files, labels = [], []
            with open(meta) as f:
                for row in csv.DictReader(f):
                    in_dev = int(row["fold"]) == split
                    if (mode == "train") != in_dev:
                        files.append(os.path.join(root, "audio", row["filename"]))
                        labels.append(int(row["target"]))
            super().__init__(files, labels, feat_type, sample_rate=44100, **kwargs)

    class TESS(_AudioFolderDataset):
        """Toronto emotional speech set: wave files named ``<speaker>_<word>_<emotion>.wav`` under ``data_dir``."""
        label_list = ["angry", "disgust", "fear", "happy", "neutral", "ps", "sad"]

        def __init__(self, mode="train", n_folds=5, split=1, feat_type="raw", archive=None, data_dir=None, **kwargs):
            import os
            root = data_dir or os.path.expanduser("~/.cache/paddle/dataset/TESS_Toronto_emotional_speech_set")
            if not os.path.isdir(root):
                raise RuntimeError(f"TESS is not available offline: expected {root}")
            wavs = sorted(os.path.join(d, f) for d, _, fs in os.walk(root) for f in fs if f.endswith(".wav"))
            files, labels = [], []
            for i, path in enumerate(wavs):
                emotion = os.path.basename(path)[:-4].split("_")[-1].lower()
                in_dev = i % n_folds + 1 == split
                if (mode == "train") != in_dev and emotion in self.label_list:
                    files.append(path)
                    labels.append(self.label_list.index(emotion))
            super().__init__(files, labels, feat_type, sample_rate=24414, **kwargs)


import sys as _sys  # noqa: E402
import types as _types  # noqa: E402


def _namespace_module(ns, name):
    m = _types.ModuleType(name)
    for k, v in vars(ns).items():
        if not k.startswith("__"):
            setattr(m, k, v.__func__ if isinstance(v, staticmethod) else v)
    _sys.modules[name] = m
    return m


_functional_ns, _features_ns = functional, features
functional = _namespace_module(functional, __name__ + ".functional")
features = _namespace_module(features, __name__ + ".features")
datasets = _namespace_module(_Datasets, __name__ + ".datasets")
backends = _namespace_module(backends, __name__ + ".backends")
