from .guidance import APG, CFG, Autoguidance, CFGPlusPlus, Guidance
from .solvers import (DDIM, DDPM, DEIS, KDPM2, LMS, PNDM, RK4, TCD, Consistency, DPMSolverMultistep, DPMSolverSDE,
                      DPMSolverSinglestep, Euler, EulerAncestral, Heun, MultiStepDPM, Solver, UniPC, SOLVERS)
from .walks import sample, walk_and_decode

def __getattr__(name):
    if name in ("FlowSDE", "FlowTrajectory", "GaussianTransition", "flow_transition"):
        from . import flow
        return getattr(flow, name)
    if name in ("generate", "Sampling", "Generation", "Sample", "Beam", "Speculative", "transform_logits"):
        from . import text
        return getattr(text, name)
    raise AttributeError(name)


__all__ = ["generate", "Sampling", "Generation", "Sample", "Beam", "Speculative", "sample", "walk_and_decode", "Solver", "SOLVERS", "Euler", "EulerAncestral", "Heun", "RK4", "KDPM2",
           "MultiStepDPM", "LMS", "DDPM", "DDIM", "PNDM", "Consistency", "TCD", "DPMSolverMultistep",
           "DPMSolverSinglestep", "DEIS", "UniPC", "DPMSolverSDE", "CFG", "CFGPlusPlus", "APG", "Autoguidance", "Guidance", "FlowSDE", "FlowTrajectory", "GaussianTransition"]
