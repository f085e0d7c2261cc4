"""Leela Chess Zero classical networks: weights-file reader, FEN input planes and batched inference
(reference: lib/core/nn/lc0.dart:1-480, lc0_proto.dart:1-583, lc0_input.dart:1-180).

* ``Lc0Reader.read_file`` gunzips a ``.pb.gz`` network and walks the protobuf wire format by hand: ``Net.weights`` (field
  10) -> input conv (1), residual blocks (2; conv1, conv2, optional SE unit), policy head (11 then 3), value head (6, FC
  7-10), optional moves-left head (12-16).  Layers are LINEAR16 (``min + v/65535 * (max-min)``), FLOAT16 or BFLOAT16.
* ``Lc0Input.from_fen`` builds the ``[1, 112, 8, 8]`` planes (current position only, side-to-move perspective).
* ``Lc0Net`` folds batch-norm into conv weights at load, keeps activations ``[B*64, C]`` (NHWC) on the device and runs
  every 3x3 / 1x1 convolution as the im2col gather kernel + tensor-core GEMM with the bias / ReLU epilogue fused;
  squeeze-excitation works on ``[B, 64, C]`` views.  ``call_batch`` returns per-position policy ``[1, P, 8, 8]`` and
  value ``[1, wdl]`` on the CPU like the reference.
"""
from __future__ import annotations

import gzip
import math
import re
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops as F
from ..nn.module import Module


# ------------------------------------------------------------------------------------------ weights ---------
@dataclass
class Lc0ConvBlock:
    weights: torch.Tensor
    biases: torch.Tensor
    bn_means: torch.Tensor
    bn_stddivs: torch.Tensor
    bn_gammas: torch.Tensor
    bn_betas: torch.Tensor


@dataclass
class Lc0SEUnit:
    w1: torch.Tensor
    b1: torch.Tensor
    w2: torch.Tensor
    b2: torch.Tensor


@dataclass
class Lc0Residual:
    conv1: Lc0ConvBlock
    conv2: Lc0ConvBlock
    se: Optional[Lc0SEUnit] = None


@dataclass
class Lc0Weights:
    filters: int
    num_blocks: int
    policy_output_planes: int
    value_filters: int
    value_fc_units: int
    input: Lc0ConvBlock
    residual: List[Lc0Residual]
    policy1: Lc0ConvBlock
    policy_out: Lc0ConvBlock
    value_conv: Lc0ConvBlock
    ip1_val_w: torch.Tensor
    ip1_val_b: torch.Tensor
    ip2_val_w: torch.Tensor
    ip2_val_b: torch.Tensor
    wdl: int
    moves_left_filters: Optional[int] = None
    moves_left_fc_units: Optional[int] = None
    moves_left_conv: Optional[Lc0ConvBlock] = None
    ip1_mov_w: Optional[torch.Tensor] = None
    ip1_mov_b: Optional[torch.Tensor] = None
    ip2_mov_w: Optional[torch.Tensor] = None
    ip2_mov_b: Optional[torch.Tensor] = None


_Field = Tuple[int, int, int, int]     # (number, wire type, start, end)


class Lc0Reader:
    @staticmethod
    def read_file(path: str) -> Lc0Weights:
        with open(path, "rb") as f:
            return Lc0Reader.read_bytes(gzip.decompress(f.read()))

    readFile = read_file

    @staticmethod
    def read_bytes(raw: bytes) -> Lc0Weights:
        d = memoryview(raw)
        wf = None
        for f in Lc0Reader._fields(d, 0, len(d)):
            if f[0] == 10:
                wf = f
        if wf is None:
            raise ValueError("lc0: no Weights (field 10) in Net message")
        return Lc0Reader._parse_weights(d, wf[2], wf[3])

    # -- protobuf wire format -----------------------------------------------------------------
    @staticmethod
    def _varint(d, i: int) -> Tuple[int, int]:
        v = shift = 0
        while True:
            b = d[i]
            i += 1
            v |= (b & 0x7F) << shift
            if not b & 0x80:
                return v, i
            shift += 7

    @staticmethod
    def _field(d, i: int) -> _Field:
        tag, j = Lc0Reader._varint(d, i)
        number, wire = tag >> 3, tag & 7
        if wire == 0:
            _, end = Lc0Reader._varint(d, j)
            return number, wire, j, end
        if wire == 1:
            return number, wire, j, j + 8
        if wire == 2:
            ln, k = Lc0Reader._varint(d, j)
            return number, wire, k, k + ln
        if wire == 5:
            return number, wire, j, j + 4
        raise ValueError(f"lc0: unknown wire type {wire} at offset {i}")

    @staticmethod
    def _fields(d, start: int, end: int):
        i = start
        while i < end:
            f = Lc0Reader._field(d, i)
            i = f[3]
            yield f

    # -- layers ---------------------------------------------------------------------------------
    @staticmethod
    def _inner_layer(d, lf: _Field) -> dict:
        raw = dict(min=0.0, max=0.0, enc=1, start=0, end=0)
        for f in Lc0Reader._fields(d, lf[2], lf[3]):
            if f[0] in (1, 2):
                if f[1] != 5:
                    raise ValueError(f"lc0: expected fixed32 (float) at field {f[0]}")
                raw["min" if f[0] == 1 else "max"] = struct.unpack_from("<f", d, f[2])[0]
            elif f[0] == 3:
                raw["start"], raw["end"] = f[2], f[3]
            elif f[0] == 4:
                if f[1] != 0:
                    raise ValueError(f"lc0: expected varint at field {f[0]}")
                raw["enc"] = Lc0Reader._varint(d, f[2])[0]
        return raw

    @staticmethod
    def _param_count(raw: dict) -> int:
        if raw["enc"] in (1, 2, 3):
            return (raw["end"] - raw["start"]) // 2
        raise ValueError(f"lc0: unsupported Layer encoding {raw['enc']}")

    @staticmethod
    def _dequantize(d, raw: dict, shape: Sequence[int]) -> torch.Tensor:
        n = Lc0Reader._param_count(raw)
        expected = int(np.prod(shape)) if len(shape) else 1
        if n != expected:
            raise ValueError(f"lc0: Layer param count {n} does not match expected shape {list(shape)} ({expected})")
        u16 = np.frombuffer(d[raw["start"]:raw["start"] + 2 * n], dtype="<u2")
        if raw["enc"] == 1:
            out = np.float32(raw["min"]) + (u16.astype(np.float64) / 65535.0 * (raw["max"] - raw["min"]))
            out = out.astype(np.float32)
        elif raw["enc"] == 2:
            out = u16.view(np.float16).astype(np.float32)
        else:
            out = (u16.astype(np.uint32) << 16).view(np.float32)
        return torch.from_numpy(np.ascontiguousarray(out)).reshape(*shape)

    @staticmethod
    def _layer(d, lf: _Field, shape) -> torch.Tensor:
        return Lc0Reader._dequantize(d, Lc0Reader._inner_layer(d, lf), shape)

    @staticmethod
    def _raw_conv_weights(d, cb: _Field) -> dict:
        for f in Lc0Reader._fields(d, cb[2], cb[3]):
            if f[0] == 1:
                return Lc0Reader._inner_layer(d, f)
        raise ValueError("lc0: ConvBlock has no weights")

    @staticmethod
    def _conv_block(d, cb: _Field, shape) -> Lc0ConvBlock:
        c_out = shape[0]
        got: Dict[int, _Field] = {}
        for f in Lc0Reader._fields(d, cb[2], cb[3]):
            if 1 <= f[0] <= 6:
                got[f[0]] = f
        if 1 not in got:
            raise ValueError("lc0: ConvBlock missing weights")

        def vec(num, default):
            return Lc0Reader._layer(d, got[num], [c_out]) if num in got else torch.full((c_out,), default)
        return Lc0ConvBlock(Lc0Reader._layer(d, got[1], shape), vec(2, 0.0), vec(3, 0.0), vec(4, 1.0), vec(5, 1.0),
                            vec(6, 0.0))

    @staticmethod
    def _se_unit(d, sf: _Field, filters: int) -> Lc0SEUnit:
        got = {f[0]: f for f in Lc0Reader._fields(d, sf[2], sf[3]) if 1 <= f[0] <= 4}
        if len(got) != 4:
            raise ValueError("lc0: SEunit missing w1/b1/w2/b2")
        w1_raw = Lc0Reader._inner_layer(d, got[1])
        n1 = Lc0Reader._param_count(w1_raw)
        hidden = n1 // filters
        if hidden * filters != n1:
            raise ValueError(f"lc0: SEunit w1 params {n1} not divisible by filters {filters}")
        return Lc0SEUnit(Lc0Reader._dequantize(d, w1_raw, [filters, hidden]), Lc0Reader._layer(d, got[2], [hidden]),
                         Lc0Reader._layer(d, got[3], [hidden, 2 * filters]), Lc0Reader._layer(d, got[4], [2 * filters]))

    @staticmethod
    def _residual(d, rf: _Field, filters: int) -> Lc0Residual:
        got = {f[0]: f for f in Lc0Reader._fields(d, rf[2], rf[3]) if 1 <= f[0] <= 3}
        if 1 not in got or 2 not in got:
            raise ValueError("lc0: residual missing conv1 or conv2")
        shape = [filters, filters, 3, 3]
        return Lc0Residual(Lc0Reader._conv_block(d, got[1], shape), Lc0Reader._conv_block(d, got[2], shape),
                           Lc0Reader._se_unit(d, got[3], filters) if 3 in got else None)

    @staticmethod
    def _parse_weights(d, start: int, end: int) -> Lc0Weights:
        one: Dict[int, _Field] = {}
        residuals: List[_Field] = []
        for f in Lc0Reader._fields(d, start, end):
            if f[0] == 2:
                residuals.append(f)
            else:
                one[f[0]] = f
        if not residuals or any(k not in one for k in (1, 3, 11, 6, 7, 8, 9, 10)):
            raise ValueError("lc0: missing required Weights fields (classical net expected)")
        n_in = Lc0Reader._param_count(Lc0Reader._raw_conv_weights(d, one[1]))
        filters = n_in // (112 * 9)
        if filters * 112 * 9 != n_in:
            raise ValueError(f"lc0: input conv weights = {n_in} does not divide 112*3*3")
        inp = Lc0Reader._conv_block(d, one[1], [filters, 112, 3, 3])
        residual = [Lc0Reader._residual(d, rf, filters) for rf in residuals]
        policy1 = Lc0Reader._conv_block(d, one[11], [filters, filters, 3, 3])
        p_planes = Lc0Reader._param_count(Lc0Reader._raw_conv_weights(d, one[3])) // (filters * 9)
        policy_out = Lc0Reader._conv_block(d, one[3], [p_planes, filters, 3, 3])
        v_filters = Lc0Reader._param_count(Lc0Reader._raw_conv_weights(d, one[6])) // filters
        value_conv = Lc0Reader._conv_block(d, one[6], [v_filters, filters, 1, 1])
        ip1_raw = Lc0Reader._inner_layer(d, one[7])
        fc_units = Lc0Reader._param_count(ip1_raw) // (v_filters * 64)
        ip1w = Lc0Reader._dequantize(d, ip1_raw, [fc_units, v_filters * 64])
        ip1b = Lc0Reader._layer(d, one[8], [fc_units])
        ip2_raw = Lc0Reader._inner_layer(d, one[9])
        wdl = Lc0Reader._param_count(ip2_raw) // fc_units
        ip2w = Lc0Reader._dequantize(d, ip2_raw, [wdl, fc_units])
        ip2b = Lc0Reader._layer(d, one[10], [wdl])
        w = Lc0Weights(filters, len(residual), p_planes, v_filters, fc_units, inp, residual, policy1, policy_out,
                       value_conv, ip1w, ip1b, ip2w, ip2b, wdl)
        if all(k in one for k in (12, 13, 14, 15, 16)):
            ml_filters = Lc0Reader._param_count(Lc0Reader._raw_conv_weights(d, one[12])) // filters
            w.moves_left_filters = ml_filters
            w.moves_left_conv = Lc0Reader._conv_block(d, one[12], [ml_filters, filters, 1, 1])
            m1 = Lc0Reader._inner_layer(d, one[13])
            ml_units = Lc0Reader._param_count(m1) // (ml_filters * 64)
            w.moves_left_fc_units = ml_units
            w.ip1_mov_w = Lc0Reader._dequantize(d, m1, [ml_units, ml_filters * 64])
            w.ip1_mov_b = Lc0Reader._layer(d, one[14], [ml_units])
            m2 = Lc0Reader._inner_layer(d, one[15])
            ml_out = Lc0Reader._param_count(m2) // ml_units
            w.ip2_mov_w = Lc0Reader._dequantize(d, m2, [ml_out, ml_units])
            w.ip2_mov_b = Lc0Reader._layer(d, one[16], [ml_out])
        return w


# -------------------------------------------------------------------------------------------- input ---------
START_FEN = "rnbqkbnr/pppppppp/8/8/8/8/PPPPPPPP/RNBQKBNR w KQkq - 0 1"
startFen = START_FEN
_PIECES = {c: i for i, c in enumerate("PNBRQKpnbrqk")}


class Lc0Input:
    @staticmethod
    def from_fen(fen: str) -> torch.Tensor:
        """``[1, 112, 8, 8]`` planes for one position without history: planes 0-5 own pieces, 6-11 opponent's (board
        flipped vertically when black is to move), 104-107 castling (own Q, own K, their Q, their K), 108 black to
        move, 109 rule-50 count, 110 zeros, 111 ones."""
        parts = re.split(r"\s+", fen.strip())
        if not parts or not parts[0]:
            raise ValueError("Lc0Input: empty FEN")
        placement = parts[0]
        stm = parts[1] if len(parts) > 1 else "w"
        castling = parts[2] if len(parts) > 2 else "-"
        try:
            rule50 = int(parts[4]) if len(parts) > 4 else 0
        except ValueError:
            rule50 = 0
        if stm not in ("w", "b"):
            raise ValueError(f'Lc0Input: side-to-move must be w or b, got "{stm}"')
        black = stm == "b"
        data = torch.zeros(112, 8, 8)
        ranks = placement.split("/")
        if len(ranks) != 8:
            raise ValueError(f"Lc0Input: expected 8 ranks in placement, got {len(ranks)}")
        for fen_rank, row in enumerate(ranks):
            rank, file = 7 - fen_rank, 0
            for ch in row:
                if ch.isdigit():
                    file += int(ch)
                    continue
                if ch not in _PIECES:
                    raise ValueError(f'Lc0Input: bad FEN char "{ch}"')
                data[_PIECES[ch], rank, file] = 1.0
                file += 1
        if black:
            own = data[6:12].flip(1).clone()
            opp = data[0:6].flip(1).clone()
            data[0:6], data[6:12] = own, opp
        wk, wq, bk, bq = ("K" in castling), ("Q" in castling), ("k" in castling), ("q" in castling)
        stm_k, stm_q, opp_k, opp_q = (bk, bq, wk, wq) if black else (wk, wq, bk, bq)
        for plane, on in ((104, stm_q), (105, stm_k), (106, opp_q), (107, opp_k)):
            if on:
                data[plane] = 1.0
        data[108] = 1.0 if black else 0.0
        data[109] = float(rule50)
        data[111] = 1.0
        return data.unsqueeze(0)

    fromFen = from_fen


# ---------------------------------------------------------------------------------------------- net ---------
@dataclass
class Lc0Output:
    policy_logits: torch.Tensor
    value: torch.Tensor

    @property
    def scalar_value(self) -> float:
        v = self.value.reshape(-1).tolist()
        return v[0] - v[2] if len(v) == 3 else v[0]

    policyLogits = property(lambda self: self.policy_logits)
    scalarValue = scalar_value


@dataclass
class _Conv:
    cin: int
    cout: int
    k: int
    w: torch.Tensor      # [Cout, k*k... ] stored [Cout, Cin*k*k] (K-major rows, the layout of a Linear weight)
    bias: torch.Tensor   # [Cout]


class Lc0Net(Module):
    BN_EPS = 1e-5

    def __init__(self, weights: Lc0Weights, device=None, dtype=torch.float32):
        super().__init__()
        self.w = weights
        self._device = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        self._dtype = dtype
        w = weights
        mk = self._make_conv
        self.input_conv = mk(w.input, 112, w.filters, 3)
        self.res_a = [mk(r.conv1, w.filters, w.filters, 3) for r in w.residual]
        self.res_b = [mk(r.conv2, w.filters, w.filters, 3) for r in w.residual]
        self.se = [None if r.se is None else self._make_se(r.se, w.filters) for r in w.residual]
        self.policy1 = mk(w.policy1, w.filters, w.filters, 3)
        self.policy_out = mk(w.policy_out, w.filters, w.policy_output_planes, 3)
        self.value_conv = mk(w.value_conv, w.filters, w.value_filters, 1)
        # value FC 1 consumes NHWC-flattened activations: permute its (c, s) columns to (s, c)
        ip1 = w.ip1_val_w.reshape(w.value_fc_units, w.value_filters, 64).permute(0, 2, 1).reshape(w.value_fc_units, -1)
        self.ip1_w, self.ip1_b = self._put(ip1), self._put(w.ip1_val_b)
        self.ip2_w, self.ip2_b = self._put(w.ip2_val_w), self._put(w.ip2_val_b)

    def _put(self, t: torch.Tensor) -> torch.Tensor:
        return t.contiguous().to(device=self._device, dtype=self._dtype)

    def _make_conv(self, cb: Lc0ConvBlock, cin: int, cout: int, k: int) -> _Conv:
        # fold batch norm: w' = w * g / sqrt(var + eps);  b' = beta - g' * (mean - b)
        new_gamma = cb.bn_gammas / torch.sqrt(cb.bn_stddivs + self.BN_EPS)
        wf = cb.weights.reshape(cout, -1) * new_gamma.reshape(cout, 1)
        bf = -new_gamma * (cb.bn_means - cb.biases) + cb.bn_betas
        return _Conv(cin, cout, k, self._put(wf), self._put(bf))

    def _make_se(self, u: Lc0SEUnit, c: int):
        hidden = u.w2.shape[0]
        return dict(w1=self._put(u.w1.t()), b1=self._put(u.b1),                      # Linear layout [hidden, C]
                    w2g=self._put(u.w2[:, :c].t()), w2b=self._put(u.w2[:, c:].t()),  # [C, hidden]
                    b2g=self._put(u.b2[:c]), b2b=self._put(u.b2[c:]), hidden=hidden)

    def parameters(self):
        return []

    # -- layers ---------------------------------------------------------------------------------------------
    def _conv(self, x, conv: _Conv, b: int, activation=None, bias: bool = True):
        """``x``: ``[B*64, Cin]`` NHWC rows -> ``[B*64, Cout]``."""
        if conv.k == 1:
            cols = x
        else:
            cols = F.im2col_nhwc(x, b, conv.cin, conv.k)
        return F.linear(cols, conv.w, conv.bias if bias else None, activation=activation)

    def _residual(self, h, i: int, b: int):
        a = self._conv(h, self.res_a[i], b, activation="relu")
        se = self.se[i]
        if se is None:
            hb = F.linear(F.im2col_nhwc(a, b, self.res_b[i].cin, 3), self.res_b[i].w, self.res_b[i].bias, residual=h)
            return F.relu(hb)
        hb = self._conv(a, self.res_b[i], b, bias=False)                  # bias enters through the SE algebra
        c = self.res_b[i].cout
        bias = self.res_b[i].bias
        pool = hb.reshape(b, 64, c).float().mean(1).to(hb.dtype) + bias   # [B, C]
        fc1 = F.linear(pool, se["w1"], se["b1"], activation="relu")
        gamma = torch.sigmoid(F.linear(fc1, se["w2g"], se["b2g"]).float()).to(hb.dtype)
        beta = F.linear(fc1, se["w2b"], se["b2b"]) + gamma * bias
        out = hb.reshape(b, 64, c) * gamma.reshape(b, 1, c) + beta.reshape(b, 1, c) + h.reshape(b, 64, c)
        return torch.relu(out).reshape(b * 64, c)

    # -- forward --------------------------------------------------------------------------------------------
    def forward_planes(self, planes: torch.Tensor):
        """``planes [B, 112, 8, 8]`` -> ``(policy [B, P, 8, 8], value [B, wdl])`` on the net's device."""
        if planes.dim() != 4 or tuple(planes.shape[1:]) != (112, 8, 8):
            raise ValueError(f"Lc0Net: expected input [B, 112, 8, 8]; got {list(planes.shape)}")
        b = planes.shape[0]
        with torch.no_grad():
            x = planes.to(device=self._device, dtype=self._dtype).permute(0, 2, 3, 1).reshape(b * 64, 112).contiguous()
            h = self._conv(x, self.input_conv, b, activation="relu")
            for i in range(len(self.res_a)):
                h = self._residual(h, i, b)
            p1 = self._conv(h, self.policy1, b, activation="relu")
            pol = self._conv(p1, self.policy_out, b)                                     # [B*64, P]
            v = self._conv(h, self.value_conv, b, activation="relu").reshape(b, -1)      # [B, 64*vf] (s, c) order
            v = F.linear(v, self.ip1_w, self.ip1_b, activation="relu")
            v = F.linear(v, self.ip2_w, self.ip2_b)
            if self.w.wdl == 3:
                v = F.softmax(v)
            p = self.w.policy_output_planes
            return pol.reshape(b, 8, 8, p).permute(0, 3, 1, 2).contiguous(), v

    def call_batch(self, inputs: Sequence[torch.Tensor]) -> List[Lc0Output]:
        if len(inputs) == 0:
            return []
        for t in inputs:
            if t.dim() != 4 or tuple(t.shape) != (1, 112, 8, 8):
                raise ValueError(f"Lc0Net.callBatch: each input must be [1, 112, 8, 8]; got {list(t.shape)}")
        pol, val = self.forward_planes(torch.cat(list(inputs), dim=0))
        pol, val = pol.float().cpu(), val.float().cpu()
        return [Lc0Output(pol[i:i + 1], val[i:i + 1]) for i in range(len(inputs))]

    callBatch = call_batch

    def forward(self, planes: torch.Tensor) -> Lc0Output:
        if planes.dim() != 4 or tuple(planes.shape) != (1, 112, 8, 8):
            raise ValueError(f"Lc0Net: expected input [1, 112, 8, 8]; got {list(planes.shape)}")
        return self.call_batch([planes])[0]
