"""Extracts the reference's golden decoder vectors for the encodings this library serves.

Run once where the reference tree is mounted:

    python tests/golden/make_golden.py <path to the nuclis source tree>

It reads inference/src/quant/fixtures/{simple,five-bit,codebook,k-affine,k-signed,iq}.json (the rows
the reference's own tests require an exact match on, inference/src/quant/decode.zig:587-592),
keeps the rows whose encoding is Q4_0 (2), Q5_0 (6), Q5_1 (7), Q8_0 (8), Q2_K (10), Q3_K (11),
Q4_K (12), Q5_K (13), Q6_K (14), IQ4_NL (20) or IQ4_XS (23), and writes
tests/golden/quant_rows.json: packed bytes as hex and expected values as the hex of
their little-endian float32 bits, so that nothing is lost to decimal printing.
The reference tree is not needed to run the tests, only to regenerate this file.
"""
import json
import os
import struct
import sys

KEEP = {2: "Q4_0", 6: "Q5_0", 7: "Q5_1", 8: "Q8_0", 10: "Q2_K", 11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K", 20: "IQ4_NL", 23: "IQ4_XS"}
FILES = ["simple.json", "five-bit.json", "codebook.json", "k-affine.json", "k-signed.json", "iq.json"]


def main(root: str) -> None:
    rows = []
    for name in FILES:
        with open(os.path.join(root, "inference/src/quant/fixtures", name)) as f:
            doc = json.load(f)
        for r in doc["rows"]:
            if r["encoding"] not in KEEP:
                continue
            values = b"".join(struct.pack("<f", v) for v in r["values"])
            # the JSON prints shortest round-trip decimals of float32 values: check that
            assert all(struct.unpack("<f", struct.pack("<f", v))[0] == v for v in r["values"])
            rows.append({
                "source": f"inference/src/quant/fixtures/{name}",
                "revision": doc["revision"],
                "encoding": r["encoding"],
                "name": KEEP[r["encoding"]],
                "bytes_hex": bytes(r["bytes"]).hex(),
                "values_f32le_hex": values.hex(),
            })
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quant_rows.json")
    with open(out, "w") as f:
        json.dump({"rows": rows}, f, indent=1)
    print(f"wrote {out}: {[(r['name'], len(r['bytes_hex']) // 2) for r in rows]}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
