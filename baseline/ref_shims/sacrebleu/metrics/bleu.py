class BLEUScore:
    pass


class BLEU:
    pass
