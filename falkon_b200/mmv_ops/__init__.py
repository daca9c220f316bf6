from .fmm import fmm
from .fmmv import fdmmv, fmmv

__all__ = ("fmm", "fmmv", "fdmmv")
