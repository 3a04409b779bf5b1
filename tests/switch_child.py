"""Child process of test_switches_gpu.py: the library reads its environment switches once per
process, so every switch setting is run in a process of its own.  Runs the named cases twice each
(the second pass replays the captured graph when graphs are on) and saves the pooler outputs."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests", "golden")):
    sys.path.insert(0, p)


def main():
    out_path, specs = sys.argv[1], sys.argv[2:]          # spec = weight_dir:is_large:case,case,...
    import cases
    from cudabert_b200.config import Engin_Config
    from cudabert_b200.cuda_model import Cuda_BERT
    result = {}
    for spec in specs:
        weight_dir, large, names = spec.split(":")
        cfg = Engin_Config()
        cfg.is_large = bool(int(large))
        cfg.model_npy_pth = weight_dir
        cfg.batch_size = cfg.max_seq_length = 0
        cfg.precision = os.environ.get("SWITCH_CHILD_PRECISION", "bf16")
        model = Cuda_BERT(0, cfg)
        for name in names.split(","):
            ids, seg, mask = cases.case_inputs(name)
            first = model.encode([ids, seg, mask])
            for _ in range(2):
                again = model.encode([ids, seg, mask])
                if not np.array_equal(first, again):
                    print("case %s: repeated passes differ" % name)
                    return 3
            result[name] = first
        model.close()
    np.savez(out_path, **result)
    return 0


if __name__ == "__main__":
    sys.exit(main())
