"""Collect the reference's own golden vectors for the inference forward path.

Run in a checkout that has the reference mounted (argument: path to the reference root).
It copies, byte for byte and SHA-256 checked, the binary fixtures that the reference's
tests/depth_one_parity.rs holds for this path:

  tests/fixtures/depth_one_main85d9d33_initial.pssa       (V7 container: RNG, init, layout)
  tests/fixtures/depth_one_main014f617_avx2_observed.bin  (f32 bit patterns; words [0,22) are the
      fresh-model chunk forward: 1 loss + 3x7 logits on ids [1,2,1] / targets [2,1,3])
  tests/fixtures/depth_one_main014f617_avx2_trained.pssa  (V7 container after two optimizer steps;
      used only as a second reader fixture)

These are data vectors produced by the reference's authors, not source code. The oracle is
checked against them in tests/test_oracle_golden.py.
"""
import hashlib
import pathlib
import shutil
import sys

FILES = {
    "depth_one_main85d9d33_initial.pssa": "29b3266df8c26ace956bf945c5092b56efcb9caf251589587d999600944ef986",
    "depth_one_main014f617_avx2_observed.bin": "f59b3a5872bed2afaa84cce668bf9d6a57569993db662ebb72aa131fa6703fbe",
    "depth_one_main014f617_avx2_trained.pssa": "69549428d1285cac528c5870559282ea93030cdfed7956721d16109cac16cf91",
}


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of the reference repository>")
    ref = pathlib.Path(sys.argv[1])
    out = pathlib.Path(__file__).resolve().parent
    for name, sha in FILES.items():
        src = ref / "tests" / "fixtures" / name
        data = src.read_bytes()
        got = hashlib.sha256(data).hexdigest()
        if got != sha:
            raise SystemExit(f"{name}: sha256 {got} differs from the value recorded by the reference ({sha})")
        shutil.copyfile(src, out / name)
        print(f"copied {name} ({len(data)} bytes)")


if __name__ == "__main__":
    main()
