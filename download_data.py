"""Fetch the public datasets and tokenizers the protocols read (needs network access; ``--dry-run`` only validates keys)."""

from __future__ import annotations

import argparse

# key -> (dataset loads, tokenizer or None)
SOURCES = {
    "wt103": ((("wikitext", "wikitext-103-raw-v1"),), None),
    "sst2": ((("glue", "sst2"),), None),
    "pythia": ((("wikitext", "wikitext-103-raw-v1"),), "EleutherAI/pythia-1.4b"),
    "gpt2": ((("wikitext", "wikitext-103-raw-v1"),), "gpt2"),
    "openwebtext": ((("openwebtext", None),), None),
}


def main(argv=None) -> dict:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--datasets", nargs="+", default=["wt103", "sst2"])
    parser.add_argument("--dry-run", action="store_true")
    args = parser.parse_args(argv)
    unknown = sorted(set(args.datasets) - set(SOURCES))
    if unknown:
        raise ValueError(f"Unknown dataset key(s): {unknown}. Known keys: {sorted(SOURCES)}")
    if args.dry_run:
        status = {"datasets": args.datasets, "status": "dry_run"}
        print(status)
        return status
    import datasets as hf_datasets

    for key in args.datasets:
        loads, tokenizer = SOURCES[key]
        for name, subset in loads:
            if name == "openwebtext":
                hf_datasets.load_dataset(name, split="train", streaming=True)
            else:
                hf_datasets.load_dataset(name, subset, split="train")
        if tokenizer:
            from transformers import AutoTokenizer

            AutoTokenizer.from_pretrained(tokenizer)
    status = {"datasets": args.datasets, "status": "available"}
    print(status)
    return status


if __name__ == "__main__":
    main()
