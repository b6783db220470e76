"""Zephyr-style DPO data: UltraFeedback-binarized with the system turn normalised, as jsonl.

    python post-training/dpo_data.py

Every conversation gets an (empty) system message in front if it has none, and only the final assistant turn of the
chosen / rejected branches is kept as the completion -- the preprocessing of the Zephyr recipe.  Output:
``data/pairwise/dpo_{train,test}_filtered.jsonl`` with keys ``chosen`` and ``rejected`` (lists of chat messages),
ready for ``preprocess_data_with_chat_template --jsonl-keys chosen rejected --only-last``.
"""
import json
import os


def normalise(example):
    prompt = [m for m in example["chosen"][:-1]]
    if not prompt or prompt[0]["role"] != "system":
        prompt.insert(0, {"role": "system", "content": ""})
    return {"chosen": prompt + example["chosen"][-1:], "rejected": prompt + example["rejected"][-1:]}


def main():
    from datasets import load_dataset
    raw = load_dataset("HuggingFaceH4/ultrafeedback_binarized")
    os.makedirs("data/pairwise", exist_ok=True)
    for name, split in (("train", "train_prefs"), ("test", "test_prefs")):
        with open(f"data/pairwise/dpo_{name}_filtered.jsonl", "w") as fh:
            for ex in raw[split]:
                fh.write(json.dumps(normalise(ex)) + "\n")


if __name__ == "__main__":
    main()
