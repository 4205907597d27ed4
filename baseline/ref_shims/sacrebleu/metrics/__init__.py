class BLEU:
    def __init__(self, *a, **k):
        raise RuntimeError("sacrebleu is not available")


class CHRF:
    def __init__(self, *a, **k):
        raise RuntimeError("sacrebleu is not available")
