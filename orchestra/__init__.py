"""``orchestra``: the public Python API of the B200 rebuild of Oxidized Neural Orchestra.

Import paths, names and signatures match the reference's module (orchestra-py/orchestra/__init__.py).
"""
from ._api import Sequential
from ._training import (PyTrainingConfig, Session, TrainedModel, all_reduce, orchestrate, parameter_server,
                        strategy_switch)

__all__ = ["PyTrainingConfig", "Sequential", "Session", "TrainedModel", "all_reduce", "orchestrate",
           "parameter_server", "strategy_switch"]
