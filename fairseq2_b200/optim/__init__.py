from fairseq2_b200.optim.adamw import AdamW
