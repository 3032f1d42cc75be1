"""``paddle.text`` (python/paddle/text/): ``viterbi_decode`` / ``ViterbiDecoder`` and dataset classes that read local
files."""
from __future__ import annotations

import torch

from .._core.tensor import as_tensor
from ..nn.layer.layers import Layer

__all__ = ["viterbi_decode", "ViterbiDecoder", "Conll05st", "Imdb", "Imikolov", "Movielens", "UCIHousing", "WMT14", "WMT16"]


def viterbi_decode(potentials, transition_params, lengths, include_bos_eos_tag=True, name=None):
    """potentials [B, T, N], transitions [N, N], lengths [B] -> (scores [B], paths [B, max_len])."""
    pot = potentials.as_subclass(torch.Tensor).float()
    trans = transition_params.as_subclass(torch.Tensor).float()
    lens = lengths.as_subclass(torch.Tensor).long()
    B, T, N = pot.shape
    max_len = int(lens.max())
    scores, paths = [], []
    for b in range(B):
        L = int(lens[b])
        alpha = pot[b, 0].clone()
        if include_bos_eos_tag:
            alpha = alpha + trans[N - 2]            # start tag = N-2 (bos), stop tag = N-1 (eos)
        back = []
        for t in range(1, L):
            m = alpha[:, None] + trans
            best, idx = torch.max(m, 0)
            alpha = best + pot[b, t]
            back.append(idx)
        if include_bos_eos_tag:
            alpha = alpha + trans[:, N - 1]
        s, last = torch.max(alpha, 0)
        path = [int(last)]
        for idx in reversed(back):
            path.append(int(idx[path[-1]]))
        path.reverse()
        scores.append(s)
        paths.append(path + [0] * (max_len - L))
    return as_tensor(torch.stack(scores)), as_tensor(torch.tensor(paths, dtype=torch.int64))


class ViterbiDecoder(Layer):
    def __init__(self, transitions, include_bos_eos_tag=True, name=None):
        super().__init__()
        self.transitions, self.include_bos_eos_tag = transitions, include_bos_eos_tag

    def forward(self, potentials, lengths):
        return viterbi_decode(potentials, self.transitions, lengths, self.include_bos_eos_tag)


def _needs_files(name):
    class _D:
        def __init__(self, data_file=None, *a, **k):
            raise RuntimeError(f"paddle.text.{name}: the corpus has to be downloaded and this build has no network; "
                               f"read your local copy with paddle.io.Dataset")
    _D.__name__ = name
    return _D


Conll05st, Imdb, Imikolov, Movielens, UCIHousing, WMT14, WMT16 = (_needs_files(n) for n in
                                                                  ("Conll05st", "Imdb", "Imikolov", "Movielens",
                                                                   "UCIHousing", "WMT14", "WMT16"))
