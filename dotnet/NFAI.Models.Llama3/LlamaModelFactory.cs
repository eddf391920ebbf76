// Drop-in replacement of NFAI.Models.Llama3/LlamaModelFactory.cs: same public surface (parameterless constructor
// that brings up the device, Dispose, TryCreate accepting general.architecture == "llama"; reference lines 15-44),
// with one CUDA context where the reference holds a Vulkan instance, device and buffer manager.
using NFAI.Core;
using NFAI.Cuda;

namespace NFAI.Models.Llama3;

public class LlamaModelFactory : AbstractModelFactory
{
    private readonly CudaContext cuda;

    // NFAI_CUDA_DEVICE selects the GPU (default 0); the reference picks the last Vulkan device it enumerates.
    public LlamaModelFactory()
    {
        var ordinal = int.TryParse(Environment.GetEnvironmentVariable("NFAI_CUDA_DEVICE"), out var v) ? v : 0;
        cuda = new CudaContext(ordinal);
    }

    public override void Dispose()
    {
        GC.SuppressFinalize(this);
        cuda.Dispose();
    }

    public override bool TryCreate(Dictionary<string, object> metadata, List<AbstractComputeCollection> tensors, ModelOptions modelOptions, out IInferenceProvider? model)
    {
        model = null;
        if (!metadata.TryGetValue("general.architecture", out var arch) || arch?.ToString() != "llama")
            return false;
        model = new LlamaModel(cuda, metadata, tensors, modelOptions.KVCacheSize);
        return true;
    }
}
