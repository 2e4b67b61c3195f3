"""Write ``urls.txt`` and ``urls_<category>.txt`` for a dataset directory (default dataset:
allenai/OLMoE-mix-0924).  Role of the reference's scripts/generate_urls.py.

    python scripts/generate_urls.py datasets/allenai_OLMoE-mix-0924 [--manifest extra.json] [--from_hub]

``--manifest``: JSON ``{category: [[prefix, first, last, zero_fill_width, extension], ...]}`` merged over
the built-in table (needed for the per-language ``starcoder`` files); ``--from_hub`` lists the files
of the hub repository instead (needs network access).
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_lm_b200 import data_prep  # noqa: E402

if __name__ == "__main__":
    p = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    p.add_argument("dataset_path")
    p.add_argument("--manifest", type=str, default=None)
    p.add_argument("--from_hub", action="store_true")
    p.add_argument("--repo_id", type=str, default="allenai/OLMoE-mix-0924")
    a = p.parse_args()
    if a.from_hub:
        urls = data_prep.urls_from_hub_listing(a.repo_id)
    else:
        manifest = dict(data_prep.OLMOE_MIX_0924)
        if a.manifest:
            with open(a.manifest) as fh:
                manifest.update(json.load(fh))
        urls = data_prep.expand_manifest(manifest)
    n = data_prep.write_url_files(a.dataset_path, urls)
    print(f"Wrote {n} URLs in {len(urls)} categories under {a.dataset_path}")
