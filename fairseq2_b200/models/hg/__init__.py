from fairseq2_b200.models.hg.adapter import (HG_FAMILY, HgCausalLMAdapter, HuggingFaceModelConfig,
                                             HuggingFaceModelError, create_hg_model, load_causal_lm,
                                             load_hg_model_simple, load_hg_tokenizer_simple, load_seq2seq_lm,
                                             register_hg_model_class, wrap_hg_model_if_causal_lm)
