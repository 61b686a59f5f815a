"""Streaming text leaves the server as the tokens' own bytes when the tokenizer is byte-level."""
import torch


def _byte_level_tokenizer(tmp_path):
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    from transformers import PreTrainedTokenizerFast
    tk = Tokenizer(models.BPE())
    tk.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tk.decoder = decoders.ByteLevel()
    tr = trainers.BpeTrainer(vocab_size=300, special_tokens=["<|endoftext|>"],
                             initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tk.train_from_iterator(["hello world", "the quick brown fox"], tr)
    fast = PreTrainedTokenizerFast(tokenizer_object=tk, eos_token="<|endoftext|>")
    fast.save_pretrained(str(tmp_path))
    return fast


def test_split_multibyte_characters_survive_token_by_token_streaming(tmp_path):
    from mstar_b200.models.tiny_model import TinyLM as TinyModel
    tok = _byte_level_tokenizer(tmp_path)
    m = TinyModel(model_dir=str(tmp_path), skip_weight_loading=True)
    assert m.tokenizer() is not None
    text = "hello wörld 你好 🎉 the fox"
    ids = tok.encode(text, add_special_tokens=False)
    assert m.decode_text(ids) == text.encode("utf-8")
    streamed = b"".join(m.decode_text([i]) for i in ids)
    assert streamed == text.encode("utf-8")
    assert "�" in "".join(tok.decode([i]) for i in ids)       # what decoding each token by itself would send
    assert m.decode_text(ids + [tok.eos_token_id]) == text.encode("utf-8")
    assert m.decode_text(torch.tensor(ids)) == text.encode("utf-8")


def test_without_a_tokenizer_ids_are_sent():
    from mstar_b200.models.tiny_model import TinyLM as TinyModel
    assert TinyModel(skip_weight_loading=True).decode_text([3, 14]) == b"3 14 "
