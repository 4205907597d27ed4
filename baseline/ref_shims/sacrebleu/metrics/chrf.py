class CHRFScore:
    pass


class CHRF:
    pass
