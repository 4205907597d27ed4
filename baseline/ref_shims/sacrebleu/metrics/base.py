class Score:
    pass
