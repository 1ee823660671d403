"""Generates tests/golden/c4_full.npz: the full-size results the GPU path is held to.

  python tests/golden/make_c4_full.py

Runs on the host cores, no GPU and no reference tree needed: oracle/cpu_engine.py (a restatement
of the reference CPU engine's execution of a memgraph, pinned against the reference interpreter's
results on the small graphs by tests/test_graphs.py) executes the 1-location memgraphs the
reference's compilers emitted, with contractions accumulated in f64 from the input values and
rounded once.  Inputs: einsummable_b200.memgraph.synthetic_llama_inputs(mg, seed=7), the ones
bench.py and the GPU tests use.

  scores            [4, 32000] f16   LLaMA-7B-shape layer forward (config 4, 2048 tokens)
  train/loss        [4] the per-sequence loss of the 4-layer training graph (config 5 shape, 2048
                    tokens).  The graph's other outputs are the updated f16 weights w - lr * grad,
                    in which the update is below half an ulp of w: they pin nothing about the
                    gradients (those are pinned at the small sizes, in f32, against the reference
                    interpreter) and are not stored.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))

from cpu_engine import cpu_engine_t  # noqa: E402
from einsummable_b200.memgraph import load_memgraph, synthetic_llama_inputs  # noqa: E402


def run(fixture):
    mg = load_memgraph(os.path.join(HERE, "graphs", fixture + ".json.gz"))
    eng = cpu_engine_t(mg, accumulate="f64")
    for k, v in synthetic_llama_inputs(mg, seed=7).items():
        eng.set_input(k, v)
    eng.run()
    return mg, eng


def main():
    out = {}
    mg, eng = run("llama7b_layer_locs1")
    out["scores"] = eng.get_output("scores")
    if "--layer-only" not in sys.argv:
        mg, eng = run("llama7b_train_l4_locs1")
        out["train/loss"] = eng.get_output("loss").astype(np.float64).reshape(-1)
    np.savez_compressed(os.path.join(HERE, "c4_full.npz"), **out)
    print("wrote c4_full.npz:", {k: v.shape for k, v in out.items() if k in ("scores", "train/loss")}, len(out), "arrays")


if __name__ == "__main__":
    main()
