"""Seeded test cases shared by the GPU parity tests and the smoke check."""
from __future__ import annotations

import numpy as np

import oracle
from lattice_b200 import synth

TOL = 1e-3     # outputs must satisfy |y - y_ref| <= TOL * (|y_ref| + rms(y_ref)) against the reference's CPU linear


def tol_ratio(y: np.ndarray, y_ref: np.ndarray) -> float:
    y = np.asarray(y, np.float64)
    y_ref = np.asarray(y_ref, np.float64)
    rms = float(np.sqrt(np.mean(y_ref ** 2)))
    return float(np.max(np.abs(y - y_ref) / (TOL * (np.abs(y_ref) + rms) + 1e-300)))


def make_case(config: int, m: int, k: int, n: int, rank: int = 0, alpha: float = 0.0, quarot: bool = False,
              bf16_x: bool = False, extra: int = 0, x_scale: float = 1.0):
    """Inputs and the oracle's answer for one projection."""
    x = synth.activations(config, m, k, extra) * np.float32(x_scale)
    if quarot:
        cols = synth.outlier_channels(config, k)
        x[:, cols] *= np.float32(20.0)
    if bf16_x:
        x = synth.bf16_round(x)
    w = synth.weights(config, n, k, extra)
    signs = None
    if quarot:
        signs = oracle.signs_from_seed(synth.QUAROT_DEFAULT_SEED, k)
        w_rot = oracle.absorb_rotation(w.astype(np.float64), n, k, signs, "input")
        payload = oracle.quantize_f64_to_q4(w_rot, symmetric=True)
    else:
        payload = oracle.quantize_f32_to_q4(w)
    lora = None
    if rank:
        a, b = synth.lora_factors(config, rank, k, n, extra)
        lora = (a, b, oracle.effective_scale(rank, alpha))
    w_deq = oracle.dequantize_q4_to_f32(payload)
    y_ref = oracle.q4_linear(x, None, m, n, k, lora=lora, rot_signs=signs, w_f32=w_deq)
    return dict(x=x, payload=payload, w_deq=w_deq, lora=lora, signs=signs, y_ref=y_ref, m=m, n=n, k=k, rank=rank)
