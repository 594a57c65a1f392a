from .decoder import Attention, Block, ModelArgs, TerraceLM, _balance_aux, _rope, rmsnorm

__all__ = ["ModelArgs", "TerraceLM", "Attention", "Block", "rmsnorm", "_rope", "_balance_aux"]
