"""Seeded synthetic inputs with the shapes, sparsity and value distributions of the five
benchmark configurations.  They stand in for the MNIST / Flickr-style data the
reference trains on (deepnet/examples/*), which is not available offline.

All arrays are float32, (dims x cases), Fortran order, from numpy's PCG64.
"""
import numpy as np


def _rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def binary_data(dims, cases, seed):
    """x_ij ~ Bernoulli(p_i), p_i ~ Beta(0.3, 2) (mean about 13 % on): configs 0, 3, 4."""
    g = _rng(seed)
    p = g.beta(0.3, 2.0, size=(dims, 1)).astype(np.float32)
    x = (g.random((dims, cases), dtype=np.float32) < p).astype(np.float32)
    return np.asfortranarray(x), p


def gaussian_data(dims, cases, seed, latent=64):
    """x = A z + 0.1 eps, standardised per dimension: config 1."""
    g = _rng(seed)
    A = g.normal(0.0, np.sqrt(1.0 / latent), size=(dims, latent))
    z = g.standard_normal((latent, cases))
    x = A @ z + 0.1 * g.standard_normal((dims, cases))
    x = (x - x.mean(axis=1, keepdims=True)) / x.std(axis=1, keepdims=True)
    return np.asfortranarray(x.astype(np.float32))


def document_counts(vocab, cases, seed, mean_len=100, zipf_s=1.07):
    """Word-count columns: length ~ Poisson(mean_len)+1, words ~ Zipf(s) over a random
    permutation of the vocabulary: config 2."""
    g = _rng(seed)
    ranks = np.arange(1, vocab + 1, dtype=np.float64)
    pw = ranks ** (-zipf_s)
    pw /= pw.sum()
    perm = g.permutation(vocab)
    lengths = g.poisson(mean_len, size=cases) + 1
    x = np.zeros((vocab, cases), dtype=np.float32, order="F")
    for j in range(cases):
        words = perm[g.choice(vocab, size=lengths[j], p=pw)]
        np.add.at(x[:, j], words, 1.0)
    return x


def weights(rows, cols, sigma, seed):
    return np.asfortranarray(_rng(seed).normal(0.0, sigma, size=(rows, cols)).astype(np.float32))
