"""Dynamically quantized layers (``lucid/nn/quantized/dynamic/__init__.py``)."""
from lucid_b200.nn.quantized.dynamic.linear import Linear, share_quantized_input
from lucid_b200.nn.quantized.dynamic.rnn import GRU, LSTM, GRUCell, LSTMCell, RNNCell

__all__ = ["Linear", "LSTM", "GRU", "LSTMCell", "GRUCell", "RNNCell", "share_quantized_input"]
