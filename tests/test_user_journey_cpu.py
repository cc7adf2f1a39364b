"""The path a user of the reference walks, end to end on CPU: text -> corpora + mixture file -> pre-training with the
recipe (checkpoints) -> DCP -> Hugging Face directory -> ``AutoModelForCausalLM(trust_remote_code)`` generation, which
must equal this package's inference engine on the same weights."""
import json
import os

import torch

from ksa_b200.config import get_preset
from ksa_b200.inference import KsaInferenceEngine
from ksa_b200.tools import build_corpus
from ksa_b200.tools.convert import convert_dcp_to_hf, hf_config_from_model_config, load_hf_checkpoint
from recipes.pretrain_ksa import get_argument_parser, train

TEMPLATE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ksa_b200", "hf")


def test_text_to_corpus_to_training_to_hf_generation(tmp_path):
    # 1. two small text sources -> corpora + a three-column mixture file (byte tokenizer: 257 ids)
    rows = {"prose": [f"the quick brown fox number {i} jumps over the lazy dog" for i in range(120)],
            "sums": [f"{i} plus {i + 1} equals {2 * i + 1}" for i in range(150)]}
    mix = tmp_path / "data" / "mix.txt"
    for name, lines in rows.items():
        src = tmp_path / f"{name}.txt"
        src.write_text("\n".join(lines) + "\n")
        info = build_corpus.main(["--input", str(src), "--output-prefix", str(tmp_path / "data" / name),
                                  "--tokenizer", "bytes", "--mix-file", str(mix), "--domain", name,
                                  "--weight", "0.5"])
        assert info["tokens"] > 64 * 40
    # 2. pre-train a tiny hybrid model on the mixture with the recipe
    cfg = get_preset("qwen3-ksa-tiny").merge({"num_layers": 2, "summary_layer_freq": [1, 0], "embed_dim": 64,
                                               "intermediate_dim": 128, "vocab_size": 257, "summary_token_begin": 257,
                                               "head_dim": 16, "summary_chunk_size": 8, "summary_sliding_chunk_num": 2})
    mc = tmp_path / "model.json"
    cfg.save(str(mc))
    ds = tmp_path / "ds.json"
    ds.write_text(json.dumps({"name": "KaiMMapDataset", "data_prefix": str(mix), "seq_length": 64, "seed": 3,
                              "global_batch_size": 2, "num_workers": 1}))
    out = tmp_path / "run"
    res = train(get_argument_parser().parse_args([
        "--model-config", str(mc), "--dataset-config", str(ds), "--output-dir", str(out), "--learning-rate", "5e-3",
        "--lr-scheduler-type", "constant", "--logging-per-step", "10", "--seed", "1", "--model-dtype", "float32",
        "--save-checkpoint-per-step", "30", "--num-training-steps", "30", "--monitor-datasource-loss"]))
    assert res["steps"] == 30 and (out / "latest").read_text() == "global_step30"
    assert res["loss"] < 4.5                                   # ln(257) = 5.55 at the start; bytes of English learn fast
    # 3. checkpoint -> Hugging Face directory
    hf_dir = convert_dcp_to_hf(str(out), "global_step30", TEMPLATE, dtype="fp32", remap="muse2hf",
                               config_overrides=hf_config_from_model_config(cfg))
    assert json.load(open(os.path.join(hf_dir, "config.json")))["vocab_size"] == 257 + cfg.summary_token_num
    # 4. generate with transformers' stock generate and with this package's engine from the same directory
    from transformers import AutoModelForCausalLM
    hf = AutoModelForCausalLM.from_pretrained(hf_dir, trust_remote_code=True, torch_dtype=torch.float32).eval()
    tok = build_corpus.ByteTokenizer()
    prompt = torch.tensor([tok.encode("the quick brown fox number 7 jumps")])
    gen = hf.generate(prompt, max_new_tokens=20, do_sample=False, eos_token_id=-1)
    model = load_hf_checkpoint(hf_dir, dtype=torch.float32)
    ours = KsaInferenceEngine(model.eval(), max_len=96, batch=1).generate(prompt, 20)
    assert torch.equal(gen, ours)
    assert gen.shape == (1, prompt.shape[1] + 20) and int(gen.max()) <= 256
