"""Write the UltraFeedback-binarized preference data as jsonl files for the three offline recipes.

    python post-training/llama_data.py

* ``data/pairwise/llama3_dpo_{train,test}_filtered.jsonl``  -- ``chosen`` / ``rejected`` conversations (DPO, reward model)
* ``data/sft/llama3_sft_{train,test}_filtered.jsonl``       -- ``messages`` = the chosen conversation
* ``data/kto/llama3_kto_{train,test}_filtered.jsonl``       -- one row per conversation with ``reward`` +1 / -1

Tokenise them with ``gpt_neox_b200.tools.datasets.preprocess_data_with_chat_template`` (``--jsonl-keys chosen rejected``
for the pairwise files, ``--jsonl-keys messages`` plus ``--reward-key reward`` for KTO).  Needs the ``datasets`` package
and network access to the Hugging Face hub.
"""
import json
import os


def write(path, rows):
    os.makedirs(os.path.dirname(path), exist_ok=True)
    with open(path, "w") as fh:
        for r in rows:
            fh.write(json.dumps(r) + "\n")


def main():
    from datasets import load_dataset
    raw = load_dataset("HuggingFaceH4/ultrafeedback_binarized")
    splits = {"train": raw["train_prefs"], "test": raw["test_prefs"]}
    for name, ds in splits.items():
        write(f"data/pairwise/llama3_dpo_{name}_filtered.jsonl", ({"chosen": r["chosen"], "rejected": r["rejected"]} for r in ds))
        write(f"data/sft/llama3_sft_{name}_filtered.jsonl", ({"messages": r["chosen"]} for r in ds))

        def kto_rows(ds=ds):
            for r in ds:
                yield {"messages": r["chosen"], "reward": 1}
                yield {"messages": r["rejected"], "reward": -1}
        write(f"data/kto/llama3_kto_{name}_filtered.jsonl", kto_rows())


if __name__ == "__main__":
    main()
