"""haste_b200: B200-native fused RNN layers (LSTM, GRU, IndRNN and LayerNorm variants)
behind the API of lmnt-com/haste's `haste_pytorch` package.

    import haste_b200 as haste
    layer = haste.LSTM(input_size=128, hidden_size=256, zoneout=0.1, dropout=0.05).cuda()
    y, (h_n, c_n) = layer(x)          # x: [T, N, C] on a B200

The compute path is libhaste_b200.so (hand-written CUDA for sm_100a behind a C ABI,
see include/haste_b200.h); build it with `python -m haste_b200.build`.
"""
from . import _C, data_parallel, ops
from .rnn import GRU, LSTM, IndRNN, LayerNormGRU, LayerNormIndRNN, LayerNormLSTM, Stack

__version__ = "0.1.0"

__all__ = ["GRU", "IndRNN", "LSTM", "LayerNormGRU", "LayerNormIndRNN", "LayerNormLSTM", "Stack",
           "data_parallel", "ops"]
