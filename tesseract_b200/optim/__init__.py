from .arena import ParamArena
from .optimizers import SGD, Adam, Optimizer

__all__ = ["ParamArena", "SGD", "Adam", "Optimizer"]
