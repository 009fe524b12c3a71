"""Tokenisers, TF-IDF, word2vec and image transforms (ghostflow-ml/src/nlp.rs, vision.rs)."""
from __future__ import annotations

import enum
import re
from collections import Counter

import numpy as np

from ._base import Estimator, out, rng_of, sigmoid, to_np


class WordTokenizer(Estimator):
    _params = ("lowercase", "min_freq", "max_vocab")

    def __init__(self):
        self._lowercase, self._min_freq, self._max_vocab = True, 1, None
        self.vocab = {"<pad>": 0, "<unk>": 1}

    def tokenize(self, text):
        return re.findall(r"\w+|[^\w\s]", text.lower() if self._lowercase else text)

    def fit(self, texts):
        c = Counter(t for s in texts for t in self.tokenize(s))
        for w, n in c.most_common(self._max_vocab):
            if n >= self._min_freq and w not in self.vocab:
                self.vocab[w] = len(self.vocab)
        self.inverse = {i: w for w, i in self.vocab.items()}
        return self

    def encode(self, text):
        return [self.vocab.get(t, 1) for t in self.tokenize(text)]

    def decode(self, ids):
        return " ".join(self.inverse.get(int(i), "<unk>") for i in ids)

    def vocab_size(self):
        return len(self.vocab)


class CharTokenizer(WordTokenizer):
    def tokenize(self, text):
        return list(text.lower() if self._lowercase else text)

    def decode(self, ids):
        return "".join(self.inverse.get(int(i), "?") for i in ids)


class BPETokenizer(Estimator):
    def __init__(self, vocab_size=1000):
        self._vocab_size, self.merges, self.vocab = vocab_size, [], {}

    def fit(self, texts):
        words = Counter(w for s in texts for w in s.lower().split())
        seqs = {w: tuple(w) + ("</w>",) for w in words}
        symbols = {c for s in seqs.values() for c in s}
        while len(symbols) + len(self.merges) < self._vocab_size:
            pairs = Counter()
            for w, s in seqs.items():
                for a, b in zip(s[:-1], s[1:]):
                    pairs[(a, b)] += words[w]
            if not pairs:
                break
            (a, b), n = pairs.most_common(1)[0]
            if n < 2:
                break
            self.merges.append((a, b))
            for w, s in seqs.items():
                res, i = [], 0
                while i < len(s):
                    if i + 1 < len(s) and s[i] == a and s[i + 1] == b:
                        res.append(a + b)
                        i += 2
                    else:
                        res.append(s[i])
                        i += 1
                seqs[w] = tuple(res)
        toks = sorted(symbols | {a + b for a, b in self.merges})
        self.vocab = {"<unk>": 0, **{t: i + 1 for i, t in enumerate(toks)}}
        self.inverse = {i: t for t, i in self.vocab.items()}
        return self

    def tokenize(self, text):
        res = []
        for w in text.lower().split():
            s = list(w) + ["</w>"]
            for a, b in self.merges:
                i, nxt = 0, []
                while i < len(s):
                    if i + 1 < len(s) and s[i] == a and s[i + 1] == b:
                        nxt.append(a + b)
                        i += 2
                    else:
                        nxt.append(s[i])
                        i += 1
                s = nxt
            res.extend(s)
        return res

    def encode(self, text):
        return [self.vocab.get(t, 0) for t in self.tokenize(text)]

    def decode(self, ids):
        return "".join(self.inverse.get(int(i), "") for i in ids).replace("</w>", " ").strip()


class TfidfVectorizer(Estimator):
    _params = ("max_features", "ngram_range", "sublinear_tf")

    def __init__(self):
        self._max_features, self._ngram_range, self._sublinear_tf = None, (1, 1), False

    def _terms(self, text):
        w = re.findall(r"\w+", text.lower())
        lo, hi = self._ngram_range
        return [" ".join(w[i:i + n]) for n in range(lo, hi + 1) for i in range(len(w) - n + 1)]

    def fit(self, texts):
        df = Counter(t for s in texts for t in set(self._terms(s)))
        terms = [t for t, _ in df.most_common(self._max_features)]
        self.vocabulary_ = {t: i for i, t in enumerate(sorted(terms))}
        n = len(texts)
        self.idf_ = np.array([np.log((1 + n) / (1 + df[t])) + 1 for t in sorted(terms)])
        return self

    def transform(self, texts):
        M = np.zeros((len(texts), len(self.vocabulary_)))
        for r, s in enumerate(texts):
            for t, c in Counter(self._terms(s)).items():
                j = self.vocabulary_.get(t)
                if j is not None:
                    M[r, j] = 1 + np.log(c) if self._sublinear_tf else c
        M *= self.idf_
        return out(M / np.maximum(np.linalg.norm(M, axis=1, keepdims=True), 1e-12))

    def fit_transform(self, texts):
        return self.fit(texts).transform(texts)


class Word2Vec(Estimator):
    """Skip-gram with negative sampling."""
    _params = ("window", "negative", "epochs", "learning_rate", "min_count", "seed")

    def __init__(self, embedding_dim=100):
        self._dim, self._window, self._negative, self._epochs, self._learning_rate = embedding_dim, 5, 5, 5, 0.025
        self._min_count, self._seed = 1, 0

    def fit(self, sentences):
        sents = [s.lower().split() if isinstance(s, str) else list(s) for s in sentences]
        c = Counter(w for s in sents for w in s)
        words = [w for w, n in c.items() if n >= self._min_count]
        self.vocab = {w: i for i, w in enumerate(words)}
        r = rng_of(self._seed)
        V = len(words)
        self.W_in = (r.random((V, self._dim)) - 0.5) / self._dim
        self.W_out = np.zeros((V, self._dim))
        p = np.array([c[w] for w in words], float) ** 0.75
        p /= p.sum()
        for _ in range(self._epochs):
            for s in sents:
                ids = [self.vocab[w] for w in s if w in self.vocab]
                for i, wi in enumerate(ids):
                    for j in range(max(0, i - self._window), min(len(ids), i + self._window + 1)):
                        if j == i:
                            continue
                        tg = np.concatenate(([ids[j]], r.choice(V, self._negative, p=p)))
                        lab = np.zeros(len(tg))
                        lab[0] = 1
                        h = self.W_in[wi]
                        g = (sigmoid(self.W_out[tg] @ h) - lab) * self._learning_rate
                        self.W_in[wi] -= g @ self.W_out[tg]
                        np.subtract.at(self.W_out, tg, g[:, None] * h[None])
        return self

    def vector(self, word):
        return out(self.W_in[self.vocab[word]])

    def most_similar(self, word, topn=5):
        v = self.W_in[self.vocab[word]]
        sims = self.W_in @ v / (np.linalg.norm(self.W_in, axis=1) * np.linalg.norm(v) + 1e-12)
        inv = {i: w for w, i in self.vocab.items()}
        return [(inv[i], float(sims[i])) for i in np.argsort(-sims) if inv[i] != word][:topn]


# ----------------------------------------------------------------------------- vision (images are [C, H, W] or [N, C, H, W])
class Interpolation(enum.Enum):
    Nearest = "nearest"
    Bilinear = "bilinear"
    Bicubic = "bicubic"


class ImageNormalization(Estimator):
    def __init__(self, mean=(0.485, 0.456, 0.406), std=(0.229, 0.224, 0.225)):
        self._mean, self._std = np.array(mean, float), np.array(std, float)

    def transform(self, img):
        a = to_np(img)
        sh = (-1, 1, 1)
        return out((a - self._mean.reshape(sh)) / self._std.reshape(sh))

    def inverse_transform(self, img):
        sh = (-1, 1, 1)
        return out(to_np(img) * self._std.reshape(sh) + self._mean.reshape(sh))

    __call__ = transform


class ImageResize(Estimator):
    _params = ("interpolation",)

    def __init__(self, width=224, height=224):
        self._width, self._height, self._interpolation = width, height, Interpolation.Bilinear

    def transform(self, img):
        import torch
        import torch.nn.functional as F
        a = torch.from_numpy(to_np(img, np.float32))
        batched = a.ndim == 4
        a = a if batched else a[None]
        mode = getattr(self._interpolation, "value", self._interpolation)
        kw = {} if mode == "nearest" else {"align_corners": False}
        r = F.interpolate(a, size=(self._height, self._width), mode=mode, **kw)
        return out((r if batched else r[0]).numpy())

    __call__ = transform


class ImageCrop(Estimator):
    def __init__(self, top=0, left=0, height=224, width=224):
        self._top, self._left, self._height, self._width = top, left, height, width

    def transform(self, img):
        return out(to_np(img)[..., self._top:self._top + self._height, self._left:self._left + self._width])

    __call__ = transform


class RandomCrop(Estimator):
    _params = ("seed", "padding")

    def __init__(self, height=32, width=32):
        self._height, self._width, self._seed, self._padding = height, width, None, 0
        self._rng = None

    def transform(self, img):
        a = to_np(img)
        if self._padding:
            a = np.pad(a, [(0, 0)] * (a.ndim - 2) + [(self._padding, self._padding)] * 2)
        self._rng = self._rng or rng_of(self._seed)
        t = int(self._rng.integers(0, a.shape[-2] - self._height + 1))
        l = int(self._rng.integers(0, a.shape[-1] - self._width + 1))
        return out(a[..., t:t + self._height, l:l + self._width])

    __call__ = transform


class ColorJitter(Estimator):
    _params = ("brightness", "contrast", "saturation", "seed")

    def __init__(self):
        self._brightness, self._contrast, self._saturation, self._seed, self._rng = 0.2, 0.2, 0.2, None, None

    def transform(self, img):
        a = to_np(img)
        self._rng = self._rng or rng_of(self._seed)
        f = lambda s: 1 + self._rng.uniform(-s, s)  # noqa: E731
        a = a * f(self._brightness)
        m = a.mean((-1, -2, -3), keepdims=True)
        a = (a - m) * f(self._contrast) + m
        g = a.mean(-3, keepdims=True)
        a = (a - g) * f(self._saturation) + g
        return out(np.clip(a, 0, 1))

    __call__ = transform


class ImageAugmentation(Estimator):
    """Pipeline: optional horizontal/vertical flip, rotation by multiples of 90 degrees, jitter, random crop."""
    _params = ("horizontal_flip", "vertical_flip", "rotate90", "color_jitter", "random_crop", "seed")

    def __init__(self):
        self._horizontal_flip, self._vertical_flip, self._rotate90 = 0.5, 0.0, False
        self._color_jitter, self._random_crop, self._seed, self._rng = None, None, None, None

    def transform(self, img):
        a = to_np(img)
        self._rng = self._rng or rng_of(self._seed)
        if self._rng.random() < self._horizontal_flip:
            a = a[..., ::-1]
        if self._rng.random() < self._vertical_flip:
            a = a[..., ::-1, :]
        if self._rotate90:
            a = np.rot90(a, int(self._rng.integers(0, 4)), axes=(-2, -1))
        t = out(np.ascontiguousarray(a))
        if self._color_jitter is not None:
            t = self._color_jitter.transform(t)
        if self._random_crop is not None:
            t = self._random_crop.transform(t)
        return t

    __call__ = transform
