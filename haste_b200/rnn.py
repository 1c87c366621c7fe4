"""`haste_pytorch`-compatible layers on top of the haste_b200 ops.

Class names, constructor keywords, parameter names/shapes/initialisation and the
`forward(input, state=None, lengths=None) -> (output, state)` contract follow the
reference's Python API (frameworks/pytorch/{base_rnn,lstm,gru,indrnn,layer_norm_lstm,
layer_norm_gru,layer_norm_indrnn}.py), so a `state_dict` saved from a reference layer
loads into the layer of the same name here.

Differences, all additive:
  * `forward` also accepts `zoneout_mask=` ([T,N,H], 1 = take the new state) and
    `dropconnect_mask=` ([H,G*H], 1 = keep the weight) so that a run can be reproduced
    exactly; without them masks are drawn as the reference draws them.
  * bfloat16 parameters/inputs are supported (fp32 accumulation inside).
  * `Stack` composes layers into multi-layer and/or bidirectional networks
    (the reference's PyTorch API has single unidirectional layers only; the
    bidirectional convention is that of its TensorFlow API, frameworks/tf/base_rnn.py:115-121).
  * The layers run on CUDA only; there is no CPU fallback.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _C, ops

__all__ = ["LSTM", "GRU", "IndRNN", "LayerNormLSTM", "LayerNormGRU", "LayerNormIndRNN", "Stack"]


def _empty_mask(x):
    return x.new_empty(0, 0, 0)


class _sm_budget:
    """While active, one persistent recurrence launch occupies at most `sms` SMs (0: no
    limit), so that the two directions of a bidirectional level are co-resident."""

    def __init__(self, sms):
        self.sms = sms

    def __enter__(self):
        if self.sms:
            _C.set_sm_budget(self.sms)

    def __exit__(self, *exc):
        if self.sms:
            _C.set_sm_budget(0)


def _bucket(ctx):
    """The flat gradient buffer of a data-parallel layer (haste_b200.data_parallel), if any."""
    return ctx.dp.bucket if ctx.dp is not None else None


def _gradients_ready(ctx, names, grads):
    """Tells the data-parallel hook that this layer's parameter gradients are queued: it
    starts their all-reduce now, while the layers below still run their backward passes."""
    if ctx.dp is not None:
        ctx.dp.gradients_ready(dict(zip(names, grads)))


# --------------------------------------------------------------------------
# autograd glue: forward saves exactly what backward needs; backward passes the
# tensors in forward layout (no permute().contiguous() copies).
# --------------------------------------------------------------------------
class _LSTMFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, training, zoneout_prob, opts, *inputs):
        dp, ctx.sm_budget = opts
        with _sm_budget(ctx.sm_budget):
            h, c, cache = ops.lstm_forward(training, zoneout_prob, *inputs)
        ctx.save_for_backward(inputs[0], *inputs[3:], h, c, cache)
        ctx.mark_non_differentiable(inputs[-1])
        ctx.training = training
        ctx.dp = dp
        return h, c

    @staticmethod
    def backward(ctx, grad_h, grad_c):
        if not ctx.training:
            raise RuntimeError('LSTM backward can only be called in training mode')
        with _sm_budget(ctx.sm_budget):
            grads = ops.lstm_backward(*ctx.saved_tensors, grad_h.contiguous(), grad_c.contiguous(),
                                      transposed=False, grads=_bucket(ctx))
        _gradients_ready(ctx, ['kernel', 'recurrent_kernel', 'bias'], grads[3:])
        return (None, None, None, *grads, None)


class _GRUFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, training, zoneout_prob, opts, *inputs):
        dp, ctx.sm_budget = opts
        with _sm_budget(ctx.sm_budget):
            h, cache = ops.gru_forward(training, zoneout_prob, *inputs)
        ctx.save_for_backward(inputs[0], *inputs[2:], h, cache)
        ctx.mark_non_differentiable(inputs[-1])
        ctx.training = training
        ctx.dp = dp
        return h

    @staticmethod
    def backward(ctx, grad_h):
        if not ctx.training:
            raise RuntimeError('GRU backward can only be called in training mode')
        with _sm_budget(ctx.sm_budget):
            grads = ops.gru_backward(*ctx.saved_tensors, grad_h.contiguous(), transposed=False, grads=_bucket(ctx))
        _gradients_ready(ctx, ['kernel', 'recurrent_kernel', 'bias', 'recurrent_bias'], grads[2:])
        return (None, None, None, *grads, None)


class _IndRNNFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, training, zoneout_prob, opts, *inputs):
        dp, ctx.sm_budget = opts
        with _sm_budget(ctx.sm_budget):
            h = ops.indrnn_forward(training, zoneout_prob, *inputs)
        ctx.save_for_backward(inputs[0], *inputs[2:], h)
        ctx.mark_non_differentiable(inputs[-1])
        ctx.training = training
        ctx.dp = dp
        return h

    @staticmethod
    def backward(ctx, grad_h):
        if not ctx.training:
            raise RuntimeError('IndRNN backward can only be called in training mode')
        with _sm_budget(ctx.sm_budget):
            grads = ops.indrnn_backward(*ctx.saved_tensors, grad_h.contiguous(), transposed=False, grads=_bucket(ctx))
        _gradients_ready(ctx, ['kernel', 'recurrent_scale', 'bias'], grads[2:])
        return (None, None, None, *grads, None)


class _LayerNormLSTMFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, training, zoneout_prob, opts, *inputs):
        dp, ctx.sm_budget = opts
        with _sm_budget(ctx.sm_budget):
            outputs = ops.layer_norm_lstm_forward(training, zoneout_prob, *inputs)
        ctx.save_for_backward(inputs[0], *inputs[3:], *outputs)
        ctx.mark_non_differentiable(inputs[-1])
        ctx.training = training
        ctx.dp = dp
        return outputs[0], outputs[1]

    @staticmethod
    def backward(ctx, grad_h, grad_c):
        if not ctx.training:
            raise RuntimeError('LayerNormLSTM backward can only be called in training mode')
        with _sm_budget(ctx.sm_budget):
            grads = ops.layer_norm_lstm_backward(*ctx.saved_tensors, grad_h.contiguous(),
                                                 grad_c.contiguous(), transposed=False, grads=_bucket(ctx))
        _gradients_ready(ctx, ['kernel', 'recurrent_kernel', 'bias', 'gamma', 'gamma_h', 'beta_h'], grads[3:])
        return (None, None, None, *grads, None)


class _LayerNormGRUFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, training, zoneout_prob, opts, *inputs):
        dp, ctx.sm_budget = opts
        with _sm_budget(ctx.sm_budget):
            output = ops.layer_norm_gru_forward(training, zoneout_prob, *inputs)
        ctx.save_for_backward(inputs[0], *inputs[2:], *output)
        ctx.mark_non_differentiable(inputs[-1])
        ctx.training = training
        ctx.dp = dp
        return output[0]

    @staticmethod
    def backward(ctx, grad_h):
        if not ctx.training:
            raise RuntimeError('LayerNormGRU backward can only be called in training mode')
        with _sm_budget(ctx.sm_budget):
            grads = ops.layer_norm_gru_backward(*ctx.saved_tensors, grad_h.contiguous(),
                                                transposed=False, grads=_bucket(ctx))
        _gradients_ready(ctx, ['kernel', 'recurrent_kernel', 'bias', 'recurrent_bias', 'gamma'], grads[2:])
        return (None, None, None, *grads, None)


class _LayerNormIndRNNFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, training, zoneout_prob, opts, *inputs):
        dp, ctx.sm_budget = opts
        with _sm_budget(ctx.sm_budget):
            output = ops.layer_norm_indrnn_forward(training, zoneout_prob, *inputs)
        ctx.save_for_backward(inputs[0], *inputs[2:], *output)
        ctx.mark_non_differentiable(inputs[-1])
        ctx.training = training
        ctx.dp = dp
        return output[0]

    @staticmethod
    def backward(ctx, grad_h):
        if not ctx.training:
            raise RuntimeError('LayerNormIndRNN backward can only be called in training mode')
        with _sm_budget(ctx.sm_budget):
            grads = ops.layer_norm_indrnn_backward(*ctx.saved_tensors, grad_h.contiguous(),
                                                   transposed=False, grads=_bucket(ctx))
        _gradients_ready(ctx, ['kernel', 'recurrent_scale', 'bias', 'gamma'], grads[2:])
        return (None, None, None, *grads, None)


# --------------------------------------------------------------------------
# state helpers (same checks and messages as the reference's base_rnn.py:79-132)
# --------------------------------------------------------------------------
def _validate_state(state, state_shape):
    if isinstance(state, (tuple, list)):
        if not isinstance(state_shape, (tuple, list)):
            raise ValueError('RNN state has invalid structure; expected {}'.format(state_shape))
        for s, ss in zip(state, state_shape):
            _validate_state(s, ss)
    else:
        shape = list(state.size())
        if len(shape) != len(state_shape):
            raise ValueError('RNN state dimension mismatch; expected {} got {}'.format(
                len(state_shape), len(shape)))
        for i, (d1, d2) in enumerate(zip(shape, state_shape)):
            if d2 is not None and d1 != d2:
                raise ValueError('RNN state size mismatch on dim {}; expected {} got {}'.format(
                    i, d2, d1))


def _zero_state(input, state_shape):
    if isinstance(state_shape, (tuple, list)) and isinstance(state_shape[0], int):
        return input.new_zeros(*state_shape)
    if isinstance(state_shape, tuple):
        return tuple(_zero_state(input, s) for s in state_shape)
    if isinstance(state_shape, list):
        return [_zero_state(input, s) for s in state_shape]
    raise ValueError('RNN state_shape is invalid')


class BaseRNN(nn.Module):
    def __init__(self, input_size, hidden_size, batch_first, zoneout, return_state_sequence):
        super().__init__()
        self.input_size = input_size
        self.hidden_size = hidden_size
        self.batch_first = batch_first
        self.zoneout = zoneout
        self.return_state_sequence = return_state_sequence
        # set by haste_b200.data_parallel.attach(): where this layer's backward pass leaves its
        # parameter gradients and how they are summed over the ranks
        self._dp = None
        # SMs one recurrence launch of this layer may occupy (0: all); Stack gives each
        # direction of a bidirectional level half of the GPU
        self._sm_budget = 0

    def _permute(self, x):
        return x.permute(1, 0, 2) if self.batch_first else x

    def _get_state(self, input, state, state_shape):
        if state is None:
            return _zero_state(input, state_shape)
        _validate_state(state, state_shape)
        return state

    def _get_final_state(self, state, lengths):
        if isinstance(state, tuple):
            return tuple(self._get_final_state(s, lengths) for s in state)
        if isinstance(state, list):
            return [self._get_final_state(s, lengths) for s in state]
        if self.return_state_sequence:
            return self._permute(state[1:]).unsqueeze(0)
        if lengths is not None:
            cols = torch.arange(state.size(1), device=state.device)
            return state[torch.as_tensor(lengths, device=state.device), cols].unsqueeze(0)
        return state[-1].unsqueeze(0)

    def _get_zoneout_mask(self, input, zoneout_mask=None):
        if zoneout_mask is not None:
            if not self.zoneout:
                raise ValueError('zoneout_mask given but the layer was built with zoneout=0')
            return zoneout_mask.to(dtype=input.dtype, device=input.device)
        if self.zoneout:
            mask = input.new_empty(input.shape[0], input.shape[1], self.hidden_size)
            mask.bernoulli_(1.0 - self.zoneout)
            return mask
        return _empty_mask(input)

    def _dropconnect(self, dropconnect_mask=None):
        """DropConnect on the recurrent matrix, applied outside the fused op exactly like
        the reference (`F.dropout(recurrent_kernel, p, training)`), so autograd carries
        the mask into the recurrent-kernel gradient."""
        R = self.recurrent_kernel
        p = getattr(self, 'dropout', 0.0)
        if not self.training or not p:
            if self._dp is not None:
                self._dp.recurrent_scale = None
            return R
        if dropconnect_mask is None:
            # drawn like F.dropout(R, p, training) draws it; kept so that the gradient summed
            # over data-parallel ranks can be scaled after the sum
            dropconnect_mask = torch.empty_like(R).bernoulli_(1.0 - p)
        scale = dropconnect_mask.to(dtype=R.dtype, device=R.device) / (1.0 - p)
        if self._dp is not None:
            self._dp.recurrent_scale = scale
        return R * scale

    def _require_cuda(self):
        flags = [p.is_cuda for p in self.parameters()]
        if any(flags) and not all(flags):
            raise ValueError('RNN tensors should all be CUDA tensors or none should be CUDA tensors')
        if not all(flags):
            raise RuntimeError('haste_b200 layers run on CUDA only; move the module with .cuda()')


def _check_rates(name, dropout, zoneout):
    if dropout is not None and (dropout < 0 or dropout > 1):
        raise ValueError('{}: dropout must be in [0.0, 1.0]'.format(name))
    if zoneout < 0 or zoneout > 1:
        raise ValueError('{}: zoneout must be in [0.0, 1.0]'.format(name))


class LSTM(BaseRNN):
    """Long Short-Term Memory layer (gate layout i,g,f,o)."""

    def __init__(self, input_size, hidden_size, batch_first=False, forget_bias=1.0, dropout=0.0,
                 zoneout=0.0, return_state_sequence=False):
        super().__init__(input_size, hidden_size, batch_first, zoneout, return_state_sequence)
        _check_rates('LSTM', dropout, zoneout)
        self.forget_bias = forget_bias
        self.dropout = dropout
        self.kernel = nn.Parameter(torch.empty(input_size, hidden_size * 4))
        self.recurrent_kernel = nn.Parameter(torch.empty(hidden_size, hidden_size * 4))
        self.bias = nn.Parameter(torch.empty(hidden_size * 4))
        self.reset_parameters()

    def to_native_weights(self):
        """Weights in torch.nn.LSTM layout: (weight_ih_l0, weight_hh_l0, bias_ih_l0, bias_hh_l0)."""
        def reorder(w):
            i, g, f, o = torch.chunk(w, 4, dim=-1)
            return torch.cat([i, f, g, o], dim=-1)
        kernel = reorder(self.kernel).permute(1, 0).contiguous()
        recurrent_kernel = reorder(self.recurrent_kernel).permute(1, 0).contiguous()
        half_bias = reorder(self.bias) / 2.0
        return (nn.Parameter(kernel), nn.Parameter(recurrent_kernel), nn.Parameter(half_bias),
                nn.Parameter(half_bias.clone()))

    def from_native_weights(self, weight_ih_l0, weight_hh_l0, bias_ih_l0, bias_hh_l0):
        """Copies torch.nn.LSTM weights into this layer."""
        def reorder(w):
            i, f, g, o = torch.chunk(w, 4, dim=-1)
            return torch.cat([i, g, f, o], dim=-1)
        self.kernel = nn.Parameter(reorder(weight_ih_l0.permute(1, 0)).contiguous())
        self.recurrent_kernel = nn.Parameter(reorder(weight_hh_l0.permute(1, 0)).contiguous())
        self.bias = nn.Parameter(reorder(bias_ih_l0 + bias_hh_l0).contiguous())

    def reset_parameters(self):
        H = self.hidden_size
        for i in range(4):
            nn.init.xavier_uniform_(self.kernel[:, i * H:(i + 1) * H])
            nn.init.orthogonal_(self.recurrent_kernel[:, i * H:(i + 1) * H])
        nn.init.zeros_(self.bias)
        nn.init.constant_(self.bias[H * 2:H * 3], self.forget_bias)

    def forward(self, input, state=None, lengths=None, zoneout_mask=None, dropconnect_mask=None):
        self._require_cuda()
        input = self._permute(input)
        shape = [1, input.shape[1], self.hidden_size]
        h0, c0 = self._get_state(input, state, (shape, shape))
        h, c = _LSTMFunction.apply(
            self.training, self.zoneout, (self._dp, self._sm_budget), input.contiguous(), h0[0].contiguous(),
            c0[0].contiguous(), self.kernel.contiguous(),
            self._dropconnect(dropconnect_mask).contiguous(), self.bias.contiguous(),
            self._get_zoneout_mask(input, zoneout_mask).contiguous())
        state = self._get_final_state((h, c), lengths)
        return self._permute(h[1:]), state


class GRU(BaseRNN):
    """Gated Recurrent Unit layer (gate layout z,r,g; reset gate applied after the
    recurrent product, as in arXiv 1406.1078v1)."""

    def __init__(self, input_size, hidden_size, batch_first=False, dropout=0.0, zoneout=0.0,
                 return_state_sequence=False):
        super().__init__(input_size, hidden_size, batch_first, zoneout, return_state_sequence)
        _check_rates('GRU', dropout, zoneout)
        self.dropout = dropout
        self.kernel = nn.Parameter(torch.empty(input_size, hidden_size * 3))
        self.recurrent_kernel = nn.Parameter(torch.empty(hidden_size, hidden_size * 3))
        self.bias = nn.Parameter(torch.empty(hidden_size * 3))
        self.recurrent_bias = nn.Parameter(torch.empty(hidden_size * 3))
        self.reset_parameters()

    def to_native_weights(self):
        """Weights in torch.nn.GRU layout: (weight_ih_l0, weight_hh_l0, bias_ih_l0, bias_hh_l0)."""
        def reorder(w):
            z, r, n = torch.chunk(w, 3, dim=-1)
            return torch.cat([r, z, n], dim=-1)
        return (nn.Parameter(reorder(self.kernel).permute(1, 0).contiguous()),
                nn.Parameter(reorder(self.recurrent_kernel).permute(1, 0).contiguous()),
                nn.Parameter(reorder(self.bias).contiguous()),
                nn.Parameter(reorder(self.recurrent_bias).contiguous()))

    def from_native_weights(self, weight_ih_l0, weight_hh_l0, bias_ih_l0, bias_hh_l0):
        """Copies torch.nn.GRU weights into this layer."""
        def reorder(w):
            r, z, n = torch.chunk(w, 3, dim=-1)
            return torch.cat([z, r, n], dim=-1)
        self.kernel = nn.Parameter(reorder(weight_ih_l0.permute(1, 0)).contiguous())
        self.recurrent_kernel = nn.Parameter(reorder(weight_hh_l0.permute(1, 0)).contiguous())
        self.bias = nn.Parameter(reorder(bias_ih_l0).contiguous())
        self.recurrent_bias = nn.Parameter(reorder(bias_hh_l0).contiguous())

    def reset_parameters(self):
        H = self.hidden_size
        for i in range(3):
            nn.init.xavier_uniform_(self.kernel[:, i * H:(i + 1) * H])
            nn.init.orthogonal_(self.recurrent_kernel[:, i * H:(i + 1) * H])
        nn.init.zeros_(self.bias)
        nn.init.zeros_(self.recurrent_bias)

    def forward(self, input, state=None, lengths=None, zoneout_mask=None, dropconnect_mask=None):
        self._require_cuda()
        input = self._permute(input)
        h0 = self._get_state(input, state, [1, input.shape[1], self.hidden_size])
        h = _GRUFunction.apply(
            self.training, self.zoneout, (self._dp, self._sm_budget), input.contiguous(), h0[0].contiguous(),
            self.kernel.contiguous(), self._dropconnect(dropconnect_mask).contiguous(),
            self.bias.contiguous(), self.recurrent_bias.contiguous(),
            self._get_zoneout_mask(input, zoneout_mask).contiguous())
        state = self._get_final_state(h, lengths)
        return self._permute(h[1:]), state


class IndRNN(BaseRNN):
    """Independently Recurrent Neural Network layer: h' = tanh(xW + u*h + b)."""

    def __init__(self, input_size, hidden_size, batch_first=False, zoneout=0.0,
                 return_state_sequence=False):
        super().__init__(input_size, hidden_size, batch_first, zoneout, return_state_sequence)
        _check_rates('IndRNN', None, zoneout)
        self.kernel = nn.Parameter(torch.empty(input_size, hidden_size))
        self.recurrent_scale = nn.Parameter(torch.empty(hidden_size))
        self.bias = nn.Parameter(torch.empty(hidden_size))
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.xavier_uniform_(self.kernel)
        nn.init.uniform_(self.recurrent_scale, -0.5, 0.5)
        nn.init.zeros_(self.bias)

    def forward(self, input, state=None, lengths=None, zoneout_mask=None):
        self._require_cuda()
        input = self._permute(input)
        h0 = self._get_state(input, state, [1, input.shape[1], self.hidden_size])
        h = _IndRNNFunction.apply(
            self.training, self.zoneout, (self._dp, self._sm_budget), input.contiguous(), h0[0].contiguous(),
            self.kernel.contiguous(), self.recurrent_scale.contiguous(), self.bias.contiguous(),
            self._get_zoneout_mask(input, zoneout_mask).contiguous())
        state = self._get_final_state(h, lengths)
        return self._permute(h[1:]), state


class LayerNormLSTM(BaseRNN):
    """LSTM with layer normalisation on x.W, h.R and the cell state."""

    def __init__(self, input_size, hidden_size, batch_first=False, forget_bias=1.0, dropout=0.0,
                 zoneout=0.0, return_state_sequence=False):
        super().__init__(input_size, hidden_size, batch_first, zoneout, return_state_sequence)
        _check_rates('LayerNormLSTM', dropout, zoneout)
        self.forget_bias = forget_bias
        self.dropout = dropout
        self.kernel = nn.Parameter(torch.empty(input_size, hidden_size * 4))
        self.recurrent_kernel = nn.Parameter(torch.empty(hidden_size, hidden_size * 4))
        self.bias = nn.Parameter(torch.empty(hidden_size * 4))
        self.gamma = nn.Parameter(torch.empty(2, hidden_size * 4))
        self.gamma_h = nn.Parameter(torch.empty(hidden_size))
        self.beta_h = nn.Parameter(torch.empty(hidden_size))
        self.reset_parameters()

    def reset_parameters(self):
        H = self.hidden_size
        for i in range(4):
            nn.init.xavier_uniform_(self.kernel[:, i * H:(i + 1) * H])
            nn.init.orthogonal_(self.recurrent_kernel[:, i * H:(i + 1) * H])
        nn.init.zeros_(self.bias)
        nn.init.constant_(self.bias[H * 2:H * 3], self.forget_bias)
        nn.init.ones_(self.gamma)
        nn.init.ones_(self.gamma_h)
        nn.init.zeros_(self.beta_h)

    def forward(self, input, state=None, lengths=None, zoneout_mask=None, dropconnect_mask=None):
        self._require_cuda()
        input = self._permute(input)
        shape = [1, input.shape[1], self.hidden_size]
        h0, c0 = self._get_state(input, state, (shape, shape))
        h, c = _LayerNormLSTMFunction.apply(
            self.training, self.zoneout, (self._dp, self._sm_budget), input.contiguous(), h0[0].contiguous(),
            c0[0].contiguous(), self.kernel.contiguous(),
            self._dropconnect(dropconnect_mask).contiguous(), self.bias.contiguous(),
            self.gamma.contiguous(), self.gamma_h.contiguous(), self.beta_h.contiguous(),
            self._get_zoneout_mask(input, zoneout_mask).contiguous())
        state = self._get_final_state((h, c), lengths)
        return self._permute(h[1:]), state


class LayerNormGRU(BaseRNN):
    """GRU with layer normalisation on x.W and h.R."""

    def __init__(self, input_size, hidden_size, batch_first=False, dropout=0.0, zoneout=0.0,
                 return_state_sequence=False):
        super().__init__(input_size, hidden_size, batch_first, zoneout, return_state_sequence)
        _check_rates('LayerNormGRU', dropout, zoneout)
        self.dropout = dropout
        self.kernel = nn.Parameter(torch.empty(input_size, hidden_size * 3))
        self.recurrent_kernel = nn.Parameter(torch.empty(hidden_size, hidden_size * 3))
        self.bias = nn.Parameter(torch.empty(hidden_size * 3))
        self.recurrent_bias = nn.Parameter(torch.empty(hidden_size * 3))
        self.gamma = nn.Parameter(torch.empty(2, hidden_size * 3))
        self.reset_parameters()

    def reset_parameters(self):
        H = self.hidden_size
        for i in range(3):
            nn.init.xavier_uniform_(self.kernel[:, i * H:(i + 1) * H])
            nn.init.orthogonal_(self.recurrent_kernel[:, i * H:(i + 1) * H])
        nn.init.zeros_(self.bias)
        nn.init.zeros_(self.recurrent_bias)
        nn.init.ones_(self.gamma)

    def forward(self, input, state=None, lengths=None, zoneout_mask=None, dropconnect_mask=None):
        self._require_cuda()
        input = self._permute(input)
        h0 = self._get_state(input, state, [1, input.shape[1], self.hidden_size])
        h = _LayerNormGRUFunction.apply(
            self.training, self.zoneout, (self._dp, self._sm_budget), input.contiguous(), h0[0].contiguous(),
            self.kernel.contiguous(), self._dropconnect(dropconnect_mask).contiguous(),
            self.bias.contiguous(), self.recurrent_bias.contiguous(), self.gamma.contiguous(),
            self._get_zoneout_mask(input, zoneout_mask).contiguous())
        state = self._get_final_state(h, lengths)
        return self._permute(h[1:]), state


class LayerNormIndRNN(BaseRNN):
    """IndRNN with layer normalisation on x.W (`gamma` is [2,H]; row 0 is used)."""

    def __init__(self, input_size, hidden_size, batch_first=False, zoneout=0.0,
                 return_state_sequence=False):
        super().__init__(input_size, hidden_size, batch_first, zoneout, return_state_sequence)
        _check_rates('LayerNormIndRNN', None, zoneout)
        self.kernel = nn.Parameter(torch.empty(input_size, hidden_size))
        self.recurrent_scale = nn.Parameter(torch.empty(hidden_size))
        self.bias = nn.Parameter(torch.empty(hidden_size))
        self.gamma = nn.Parameter(torch.empty(2, hidden_size))
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.xavier_uniform_(self.kernel)
        nn.init.uniform_(self.recurrent_scale, -0.5, 0.5)
        nn.init.zeros_(self.bias)
        nn.init.ones_(self.gamma)

    def forward(self, input, state=None, lengths=None, zoneout_mask=None):
        self._require_cuda()
        input = self._permute(input)
        h0 = self._get_state(input, state, [1, input.shape[1], self.hidden_size])
        h = _LayerNormIndRNNFunction.apply(
            self.training, self.zoneout, (self._dp, self._sm_budget), input.contiguous(), h0[0].contiguous(),
            self.kernel.contiguous(), self.recurrent_scale.contiguous(), self.bias.contiguous(),
            self.gamma.contiguous(), self._get_zoneout_mask(input, zoneout_mask).contiguous())
        state = self._get_final_state(h, lengths)
        return self._permute(h[1:]), state


_reversed_index = {}


class _FlipTime(torch.autograd.Function):
    """Time reversal of a `[T, ...]` tensor as a row gather (whole `[N, F]` slabs copied with
    wide accesses; `torch.flip`'s element-indexed kernel runs at a fifth of the copy bandwidth
    on these shapes).  Its gradient is the same reversal."""

    @staticmethod
    def forward(ctx, x):
        return _flip_rows(x)

    @staticmethod
    def backward(ctx, g):
        return _flip_rows(g)


def _flip_rows(x):
    T = x.shape[0]
    key = (T, x.device)
    idx = _reversed_index.get(key)
    if idx is None:
        idx = _reversed_index[key] = torch.arange(T - 1, -1, -1, device=x.device)
    return x.contiguous().index_select(0, idx)


def _flip_time(x):
    return _FlipTime.apply(x)


class Stack(nn.Module):
    """`num_layers` layers of one cell type, optionally bidirectional.

    Time-major input `[T,N,C]`.  A bidirectional level runs a forward layer on the
    sequence and a second layer on the time-reversed sequence, reverses that layer's
    output back, and feeds `cat([fw, bw], -1)` to the next level; the two directions
    of a level are issued on two CUDA streams, and (`concurrent_directions`, the default)
    each direction's persistent recurrence kernel is limited to half of the GPU's SMs so that
    the two are co-resident and really run at the same time.
    Returns the last level's output (`[T,N,H]` or `[T,N,2H]`).
    `masks`, if given, is a list (per level) of lists (per direction) of dicts with
    optional keys `zoneout_mask` / `dropconnect_mask`.
    """

    def __init__(self, cell, input_size, hidden_size, num_layers=1, bidirectional=False,
                 concurrent_directions=True, **cell_kwargs):
        super().__init__()
        self.bidirectional = bidirectional
        self.concurrent_directions = concurrent_directions
        self.num_layers = num_layers
        dirs = 2 if bidirectional else 1
        layers = []
        for l in range(num_layers):
            in_size = input_size if l == 0 else hidden_size * dirs
            layers.append(nn.ModuleList([cell(in_size, hidden_size, **cell_kwargs)
                                         for _ in range(dirs)]))
        self.layers = nn.ModuleList(layers)
        self._side = None
        self._budget_set = False

    def forward(self, x, masks=None):
        for l, level in enumerate(self.layers):
            kw = masks[l] if masks is not None else [{} for _ in level]
            if not self.bidirectional:
                x, _ = level[0](x, **kw[0])
                continue
            if self._side is None:
                self._side = torch.cuda.Stream(device=x.device)
            if not self._budget_set and self.concurrent_directions:
                # half of the GPU per direction: the two directions' persistent kernels, issued
                # on two streams, then run at the same time instead of one after the other
                sms = torch.cuda.get_device_properties(x.device).multi_processor_count // 2
                for lv in self.layers:
                    for layer in lv:
                        layer._sm_budget = sms
                self._budget_set = True
            main = torch.cuda.current_stream()
            # the side stream starts after everything queued so far (x included) and makes its
            # own reversed copy, so no kernel of the backward-direction layer can run ahead
            # of the flip that produces its input
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                x.record_stream(self._side)
                x_rev = _flip_time(x)
                y_bw, _ = level[1](x_rev, **kw[1])
                y_bw = _flip_time(y_bw)
            y_fw, _ = level[0](x, **kw[0])
            main.wait_stream(self._side)
            y_bw.record_stream(main)
            x = torch.cat([y_fw, y_bw], dim=-1)
        return x
