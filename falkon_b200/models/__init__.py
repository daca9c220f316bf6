from .falkon import Falkon

__all__ = ("Falkon",)
