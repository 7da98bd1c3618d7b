"""Command line of the exporter, with the reference's flags and report (export.py:15-61):

    python -m nativebit_b200.export --checkpoint ckpt.pt --output model.nbpack [--verify] [--device cuda:0]

The nearest-entry search and the bit-packing run on the GPU; the file written is the reference's .nbpack.
"""
from __future__ import annotations

import argparse
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Export a NativeBit training checkpoint to the packed format")
    ap.add_argument("--checkpoint", required=True, help="training checkpoint (.pt)")
    ap.add_argument("--output", required=True, help="packed output (.nbpack)")
    ap.add_argument("--verify", action="store_true", help="compare the packed model's logits with the checkpoint's")
    ap.add_argument("--device", default="cuda", help="CUDA device that quantises and packs (default: cuda)")
    args = ap.parse_args(argv)
    from .pack import export_packed, verify_packed

    print(f"Exporting: {args.checkpoint}\nOutput:    {args.output}\n")
    st = export_packed(args.checkpoint, args.output, args.device)
    print(f"Original checkpoint:  {st['original_size_bytes'] / 2**20:.1f} MB")
    print(f"Packed file:          {st['file_size_bytes'] / 2**20:.1f} MB")
    print(f"Compression ratio:    {st['compression_ratio']:.1f}x")
    print(f"Bit width:            {st['bits']}-bit")
    print(f"Quantized layers:     {st['n_quantized_layers']}\n")
    print(f"  Packed indices:     {st['packed_indices_bytes'] / 1024:.1f} KB")
    print(f"  Codebook tables:    {st['codebook_bytes'] / 1024:.1f} KB")
    print(f"  Float params:       {st['float_param_bytes'] / 1024:.1f} KB")
    if args.verify:
        print("\nVerifying packed model...")
        res = verify_packed(args.checkpoint, args.output, args.device)
        print(f"  Max logit diff:   {res['max_diff']:.6f}")
        print(f"  Mean logit diff:  {res['mean_diff']:.6f}")
        print(f"  Status:           {'PASS' if res['passed'] else 'FAIL'}")
        if not res["passed"]:
            return 1
    print("\nDone.")
    return 0


if __name__ == "__main__":
    sys.exit(main())
