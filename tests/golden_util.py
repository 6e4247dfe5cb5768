"""Helpers shared by the CPU and GPU tests for the committed golden fixtures."""
import json
import os

import numpy as np

import glm_tail

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
MODEL_FIXTURES = ["glm_model", "glm_ptuning_v2_model", "glm2_model", "glm3_model", "glm3_ptuning_v2_model",
                  "glm4_model"]
GOLDEN_ATOL = 5e-4  # the reference's own tolerance for these vectors (chatglm_test.cpp:338,350,360)


def load_fixture(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    meta = json.loads(str(z["meta"]))
    w = {k[2:]: z[k] for k in z.files if k.startswith("w_")}
    return z, meta, w


def steps(z):
    for i in (1, 2, 3):
        yield i, z[f"x{i}"], z[f"y{i}"], z[f"qkv{i}"], z[f"ctx{i}"], int(z[f"n_past{i}"])


def model_output(meta, w, x, ctx):
    state, _ = glm_tail.pre(meta["family"], w, x)
    return glm_tail.post(meta["family"], w, state, ctx)
