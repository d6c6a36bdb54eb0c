"""spite_b200: a small, whole inference engine for one B200 (sm_100a), built
after giveen/spite's Llama 4 path: configuration, weights, layers made of parts,
a paged cache, one step function, a scheduler, sampling, and trace replay."""

__version__ = "0.1.0"

from . import config, parts  # noqa: F401  (registers the built-in architecture and parts)


def __getattr__(name):
    if name in ("LLM", "generate"):
        from . import api
        return getattr(api, name)
    raise AttributeError(name)
