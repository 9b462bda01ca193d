"""Shared helpers for the parity tests: golden loading and model/oracle weight construction."""
from __future__ import annotations

import os

import numpy as np
import torch

from tests import golden_inputs as gi

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden(name: str):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def build_model(spec):
    """Our MathLM with the spec's seeded init + perturbation (bit-identical to the reference's; the golden file
    carries the digest of the reference's weights)."""
    from ultraviolet_b200.model import MathLM, make_config
    torch.manual_seed(spec["seed"])
    m = MathLM(make_config(spec["preset"], **spec["over"]))
    gi.perturb_(m, spec)
    return m


def oracle_weights(m, round_to="fp32"):
    from oracle import model as om
    params = {k: v.detach().float().numpy() for k, v in m.state_dict().items()}
    if round_to != "fp32":
        params = {k: om.ROUNDERS[round_to](v) for k, v in params.items()}
    return om.fuse_weights(params, m.cfg, round_to)
