// One CUDA device: stands where (Vk, Device, VulkanBufferManager) stand in the reference
// (NFAI.Models.Llama3/LlamaModelFactory.cs:9-22).
namespace NFAI.Cuda;

public sealed class CudaContext : IDisposable
{
    internal IntPtr Handle;

    public CudaContext(int deviceOrdinal = 0)
    {
        Native.Check(Native.nfai_ctx_create(deviceOrdinal, out Handle), IntPtr.Zero);
    }

    public void Dispose()
    {
        if (Handle != IntPtr.Zero) { Native.nfai_ctx_destroy(Handle); Handle = IntPtr.Zero; }
        GC.SuppressFinalize(this);
    }
}
