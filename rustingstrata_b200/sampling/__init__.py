from .sampler import Sampler, SamplingParams, SamplingError, XorShift64, seed_state, NON_FINITE
