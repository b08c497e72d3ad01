"""Generate the whole-model golden files of the reference's parity gate under tests/golden/parity_audit*/.

    python tests/golden/make_parity_audit_golden.py --reference /path/to/transformer-cuda

Calls the reference's own `pytorch_src.utils.generate_golden_reference` (seed 42) unmodified. It writes
config.txt, pytorch_params.bin, inputs.bin, targets.bin, pytorch_logits.bin, pytorch_loss.bin and
pytorch_grads.bin - the files that the reference's src/parity_audit.cu reads and that
scripts/compare_parity.py:108-117 compares the CUDA model against (logits, loss <= 1e-5; grads <= 5e-5).
Two shapes: the script's default (B=4,T=16,C=64,L=2,H=4,V=65; d_head=16) and one with d_head=64
(B=2,T=48,C=128,L=1,H=2,V=65) so that the BF16 tensor-core mode can be run through the same model.
"""
import argparse
import os
import sys

CASES = {
    "parity_audit": dict(batch_size=4, seq_len=16, d_model=64, num_layers=2, num_heads=4, vocab_size=65, seed=42),
    "parity_audit_d64": dict(batch_size=2, seq_len=48, d_model=128, num_layers=1, num_heads=2, vocab_size=65, seed=42),
}

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of a transformer-cuda checkout")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from pytorch_src.utils import generate_golden_reference

    here = os.path.dirname(os.path.abspath(__file__))
    for name, kw in CASES.items():
        generate_golden_reference(output_dir=os.path.join(here, name), **kw)
