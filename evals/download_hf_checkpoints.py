"""Download every revision (``main`` and the ``step*`` branches) of a hub model, e.g. the intermediate
checkpoints of allenai/OLMoE-1B-7B-0924, for evaluation next to one's own run.  Needs network access.

    python evals/download_hf_checkpoints.py --model_choice allenai/OLMoE-1B-7B-0924 --out_dir hf_checkpoints [--every 10]
"""
import argparse
import os

if __name__ == "__main__":
    p = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    p.add_argument("--model_choice", type=str, default="allenai/OLMoE-1B-7B-0924")
    p.add_argument("--out_dir", type=str, default="hf_checkpoints")
    p.add_argument("--every", type=int, default=1, help="keep every n-th step checkpoint")
    a = p.parse_args()
    from huggingface_hub import list_repo_refs, snapshot_download

    branches = [b.name for b in list_repo_refs(a.model_choice).branches]
    steps = sorted((b for b in branches if b.startswith("step")), key=lambda x: int(x.split("-")[0][4:]))[::a.every]
    revisions = (["main"] if "main" in branches else []) + steps
    root = os.path.join(a.out_dir, a.model_choice.replace("/", "__"))
    os.makedirs(root, exist_ok=True)
    with open(os.path.join(root, "checkpoints.txt"), "w") as fh:
        fh.write("\n".join(revisions) + "\n")
    for rev in revisions:
        snapshot_download(repo_id=a.model_choice, revision=rev, local_dir=os.path.join(root, rev))
