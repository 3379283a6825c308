from .base import (Aux, EMASpec, Exponentiated, Mean, Metric, Moments, Objective, Ratio, Step, Summed, Weighted, pool)

__all__ = ["Aux", "EMASpec", "Exponentiated", "Mean", "Metric", "Moments", "Objective", "Ratio", "Step", "Summed",
           "Weighted", "pool", "DiffusionObjective", "LMObjective", "JepaObjective", "Supervised"]


def __getattr__(name):
    if name == "DiffusionObjective":
        from .diffusion import DiffusionObjective
        return DiffusionObjective
    if name in ("LMObjective", "Perplexity"):
        from . import lm
        return getattr(lm, name)
    if name == "JepaObjective":
        from .jepa import JepaObjective
        return JepaObjective
    if name in ("Alignment", "AlignedDiffusionObjective", "GuidanceDistillationObjective", "Projector", "spatial_zscore"):
        from . import diffusion_extras
        return getattr(diffusion_extras, name)
    if name == "EndToEndObjective":
        from .end_to_end import EndToEndObjective
        return EndToEndObjective
    if name == "NodePerturbation":
        from .perturbation import NodePerturbation
        return NodePerturbation
    if name in ("AdversarialDistillationObjective",):
        from . import adversarial
        return getattr(adversarial, name)
    if name in ("ExpertBalance", "refuse_fixed_routers", "UntrainedRouter"):
        from . import routing
        return getattr(routing, name)
    if name == "Supervised":
        from .supervised import Supervised
        return Supervised
    raise AttributeError(name)
