from .falkon import Falkon, InCoreFalkon

__all__ = ("Falkon", "InCoreFalkon")
