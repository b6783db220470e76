#!/usr/bin/env python
"""Upload a converted model directory to the Hugging Face hub (``tools/ckpts/upload.py`` of the reference).
Needs network access and ``huggingface_hub``; ``python -m gpt_neox_b200.tools.ckpts.upload <repo> <branch> <dir>``."""
import os
import sys


def main(argv=None):
    argv = argv or sys.argv[1:]
    if len(argv) != 3:
        print("usage: upload.py <hf-repo-name> <branch-name> <folder>")
        return 2
    from huggingface_hub import HfApi, create_repo
    repo, branch, folder = argv
    try:
        create_repo(repo, repo_type="model")
    except Exception:
        print("repo already exists (or cannot be created), uploading into it")
    api = HfApi()
    files = [f for f in os.listdir(folder) if f.endswith((".bin", ".safetensors", ".json", ".txt", ".model"))]
    for f in files:
        print(f"Uploading {f} to {repo}...")
        api.upload_file(path_or_fileobj=os.path.join(folder, f), path_in_repo=f, repo_id=repo, repo_type="model",
                        commit_message=f"Upload {f}", revision=branch)
    return 0


if __name__ == "__main__":
    sys.exit(main())
