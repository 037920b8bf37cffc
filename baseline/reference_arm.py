"""Reference arm of the benchmark: runs the unmodified reference installed under baseline/_ref."""
import json
import os


def run(opts, model, layouts, samples_per_gpu, micro_batch, vocab):
    rank = int(os.environ.get("RANK", "0"))
    here = os.path.dirname(os.path.abspath(__file__))
    if not os.path.isdir(os.path.join(here, "_ref")):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed"}), flush=True)
        return
    if rank == 0:
        print(json.dumps({"impl": "reference", "unavailable": "reference runner not wired yet"}), flush=True)
