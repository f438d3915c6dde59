class Attention:  # placeholders used only in isinstance checks / annotations
    pass


class GroupedQueryAttention:
    pass


class TransformerBlock:
    pass
