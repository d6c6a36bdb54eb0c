"""spite_b200: a small, whole inference engine for one B200 (sm_100a), built
after giveen/spite's Llama 4 path: configuration, weights, layers made of parts,
a paged cache, one step function, a scheduler, sampling, and trace replay."""

__version__ = "0.1.0"
