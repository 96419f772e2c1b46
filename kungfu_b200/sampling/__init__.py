from .sampler import CANDIDATES, Candidates, Rng, Sampling, argmax, draw, sample, sample_sparse
