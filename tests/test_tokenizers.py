"""A ``model_dir`` with Hugging Face tokenizer files makes the models tokenise with it (ids, chat template, decoded
text output); without one they fall back to byte-level ids."""
import pytest
import torch


def _save_tokenizer(path, chat_template=True):
    tokenizers = pytest.importorskip("tokenizers")
    from transformers import PreTrainedTokenizerFast
    words = ["[UNK]", "<|user|>", "<|assistant|>", "hello", "world", "a", "red", "fox", "say", "hi"]
    tok = tokenizers.Tokenizer(tokenizers.models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="[UNK]"))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.WhitespaceSplit()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="[UNK]")
    if chat_template:
        fast.chat_template = ("{% for m in messages %}<|user|> {{ m['content'] }} {% endfor %}"
                              "{% if add_generation_prompt %}<|assistant|>{% endif %}")
    fast.save_pretrained(str(path))


def test_models_use_the_checkpoints_tokenizer_when_there_is_one(tmp_path):
    from mstar_b200.models.qwen3_omni import Qwen3OmniModel
    from mstar_b200.models.wan22 import Wan22Model
    _save_tokenizer(tmp_path / "tokenizer")               # diffusers-style sub-directory
    m = Wan22Model(model_dir=str(tmp_path), skip_weight_loading=True, small=True)
    assert m.tokenizer() is not None
    assert m.encode_text("a red fox", 1000) == [5, 6, 7]
    ids = m.process_prompt("a red fox", ["text"], ["video"], {})["input_ids"][0].tolist()
    assert ids[:3] == [5, 6, 7]
    d2 = tmp_path / "llm"
    d2.mkdir()
    _save_tokenizer(d2)
    q = Qwen3OmniModel(model_dir=str(d2), skip_weight_loading=True, small=True)
    ids = q.process_prompt("say hi", ["text"], ["text"], {})["input_ids"][0].tolist()
    assert [1, 8, 9, 2] == [i for i in ids if i in (1, 2, 8, 9)]        # user tag, the words, the assistant tag
    assert q.postprocess(torch.tensor([3, 4]), "text", {}) == b"hello world"


def test_models_fall_back_to_bytes_without_tokenizer_files(tmp_path):
    from mstar_b200.models.qwen3_omni import Qwen3OmniModel
    q = Qwen3OmniModel(model_dir=None, skip_weight_loading=True, small=True)
    assert q.tokenizer() is None
    assert q.encode_text("hi", 5000, 1000) == [104, 105]
    assert q.postprocess(torch.tensor([3, 4]), "text", {}) == b"3 4 "
    q2 = Qwen3OmniModel(model_dir=str(tmp_path), skip_weight_loading=True, small=True)      # a directory without files
    assert q2.tokenizer() is None
