from .conjgrad import ConjugateGradient, FalkonConjugateGradient, Optimizer, StopOptimizationException

__all__ = ("Optimizer", "ConjugateGradient", "FalkonConjugateGradient", "StopOptimizationException")
