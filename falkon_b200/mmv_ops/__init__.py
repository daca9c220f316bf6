from .fmmv import fdmmv, fmmv

__all__ = ("fmmv", "fdmmv")
