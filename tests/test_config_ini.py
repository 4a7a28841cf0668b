"""The config.ini reader against files written the way the reference's converter writes them
(tools/FT_convert_weight_to_bin_final.py:43-64: Python's configparser, section [llama]).  CPU only."""
import configparser
import os

import pytest


def _write(path, **overrides):
    cfg = configparser.ConfigParser()
    cfg["llama"] = {}
    values = {"model_name": "llama-2-7b-chat", "head_num": "32", "kv_head_num": "32", "hidden_size": "4096", "head_size": "128",
              "inter_size": "11008", "num_layer": "32", "vocab_size": "32000", "bos_token_id": "1", "eos_token_id": "2",
              "weight_data_type": "fp16", "max_position_embeddings": "4096", "rope_theta": "10000.0", "rms_norm_eps": "1e-05",
              "attention_bias": "False", "top_k": "50"}
    values.update(overrides)
    for k, v in values.items():
        if v is not None:
            cfg["llama"][k] = v
    with open(path, "w") as f:
        cfg.write(f)


def test_reads_what_the_converter_writes(ob, tmp_path):
    p = os.path.join(str(tmp_path), "config.ini")
    _write(p)
    cfg, top_k = ob.llama_config_from_ini(p, max_batch=8, max_seq_len=2048, tp_rank=3, tp_size=8)
    assert (cfg.num_layers, cfg.hidden, cfg.head_num, cfg.kv_head_num, cfg.head_size, cfg.inter_size, cfg.vocab_size) == \
        (32, 4096, 32, 32, 128, 11008, 32000)
    assert (cfg.bos_id, cfg.eos_id, cfg.attn_bias, top_k) == (1, 2, 0, 50)
    assert cfg.rope_base == 10000.0 and abs(cfg.rms_eps - 1e-5) < 1e-12
    assert (cfg.max_batch, cfg.max_seq_len, cfg.tp_rank, cfg.tp_size) == (8, 2048, 3, 8)   # the caller's, not the file's
    cfg, _ = ob.llama_config_from_ini(p)                                                     # no cache length given
    assert cfg.max_seq_len == 4096
    _write(p, attention_bias="True", kv_head_num="8", rope_theta="500000.0", top_k=None)
    cfg, top_k = ob.llama_config_from_ini(p)
    assert (cfg.attn_bias, cfg.kv_head_num, cfg.rope_base, top_k) == (1, 8, 500000.0, 0)


@pytest.mark.parametrize("overrides,needle", [
    ({"head_num": None}, "head_num"), ({"num_layer": "thirty-two"}, "num_layer"), ({"hidden_size": "4000"}, "hidden_size"),
    ({"attention_bias": "maybe"}, "attention_bias"), ({"weight_data_type": "int8"}, "weight_data_type"),
])
def test_reports_the_key_that_is_wrong(ob, tmp_path, overrides, needle):
    p = os.path.join(str(tmp_path), "config.ini")
    _write(p, **overrides)
    with pytest.raises(ob.OnellmError) as e:
        ob.llama_config_from_ini(p)
    assert e.value.status == -5 and needle in str(e.value)


def test_missing_file_and_section(ob, tmp_path):
    with pytest.raises(ob.OnellmError) as e:
        ob.llama_config_from_ini(os.path.join(str(tmp_path), "nope.ini"))
    assert e.value.status == -5
    p = os.path.join(str(tmp_path), "other.ini")
    with open(p, "w") as f:
        f.write("[gpt]\nhead_num = 12\n")
    with pytest.raises(ob.OnellmError) as e:
        ob.llama_config_from_ini(p)
    assert "[llama]" in str(e.value)
