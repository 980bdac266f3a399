from .standard import StandardCombineInput, StandardDispatcher, StandardDispatchOutput, StandardTopKOutput

__all__ = ["StandardCombineInput", "StandardDispatcher", "StandardDispatchOutput", "StandardTopKOutput"]
