"""tokenomos_b200: a small, whole inference engine for the LFM3 hybrid conv decoder on one
NVIDIA B200 (sm_100a): typed config and registry, weights by tensor name, parts, cache manager,
one step function, scheduler, sampling, Python and command-line entry points, trace replay."""

__all__ = ["LLM", "SamplingParams"]


def __getattr__(name):
    if name in __all__:
        from tokenomos_b200.api import llm
        return getattr(llm, name)
    raise AttributeError(name)
