from .sampler import (DEFAULT_SEED, SampleRow, Sampler, SamplingParams, lcg_advance,
                      run_sampling_params)

__all__ = ["DEFAULT_SEED", "SampleRow", "Sampler", "SamplingParams", "lcg_advance", "run_sampling_params"]
