from .sampler import CANDIDATES, RING, STATE_WORDS, Sampling, generator_state, pack_state
