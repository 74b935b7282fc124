"""The two reference networks (machine_learning/src/models.rs:19-263, benchmarks/issue/suites.py:148-178).

    nielsen():  conv 20@5x5 -> max-pool 2 -> dense 100 sigmoid -> dense 10 softmax
    lenet5():   conv 6@5x5 pad 2 tanh -> pool 2 -> conv 16@5x5 tanh -> pool 2 -> dense 120/84 tanh -> dense 10 softmax
"""
from orchestra import Sequential
from orchestra.activations import Sigmoid, Softmax, Tanh
from orchestra.arch import Conv2d, Dense, MaxPooling
from orchestra.initialization import Xavier


def nielsen() -> Sequential:
    return Sequential([
        Conv2d((1, 28, 28), (20, 1, 5), 1, 0, Xavier()),
        MaxPooling((20, 24, 24), 2, 2, 0),
        Dense(100, Xavier(), Sigmoid()),
        Dense(10, Xavier(), Softmax()),
    ])


def lenet5() -> Sequential:
    return Sequential([
        Conv2d((1, 28, 28), (6, 1, 5), 1, 2, Xavier(), Tanh()),
        MaxPooling((6, 28, 28), 2, 2, 0),
        Conv2d((6, 14, 14), (16, 6, 5), 1, 0, Xavier(), Tanh()),
        MaxPooling((16, 10, 10), 2, 2, 0),
        Dense(120, Xavier(), Tanh()),
        Dense(84, Xavier(), Tanh()),
        Dense(10, Xavier(), Softmax()),
    ])
