from .bpe import ByteLevelBPE, TokenizerError

__all__ = ["ByteLevelBPE", "TokenizerError"]
