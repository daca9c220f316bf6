from .flk_preconditioner import FalkonPreconditioner, Preconditioner

__all__ = ("Preconditioner", "FalkonPreconditioner")
