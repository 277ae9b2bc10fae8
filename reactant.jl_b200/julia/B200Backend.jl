# B200Backend.jl -- binds Reactant.jl's PJRT wrapper structs to librx_b200.so.
#
# Written against Reactant.jl v0.2.280 (src/xla/PJRT/*.jl, src/xla/XLA.jl,
# src/accelerators/Registration.jl).  Julia is not installed where the engine
# is built, so this file has not been executed there; every call it makes is
# exercised from Python through the same C ABI in the test suite.
module B200Backend

using Reactant: Reactant, XLA, MLIR
using Reactant.XLA: PJRT
using Libdl

const lib = Ref{Ptr{Cvoid}}(C_NULL)
sym(name) = Libdl.dlsym(lib[], name)

function __init__()
    lib[] = Libdl.dlopen(get(ENV, "RX_B200_LIB", "librx_b200.so"))
    # Runtime failures are reported through the slot Reactant installs its throwing
    # callback in (src/xla/XLA.jl:203-204, deps/ReactantExtra/API.cpp:262).
    unsafe_store!(
        Ptr{Ptr{Cvoid}}(sym(:ReactantThrowError)),
        @cfunction(XLA.reactant_err, Cvoid, (Cstring,)),
    )
    # Take precedence over the stock CUDA registration (src/accelerators/GPU.jl:71-92).
    Reactant.Accelerators.register_backend(
        "b200"; priority=600, pjrt_initialize_function=make_client, platform="cuda"
    )
    return nothing
end

# MakeGPUClient keeps the reference signature (API.cpp:528-582).
function make_client(;
    node_id::Integer=0,
    num_nodes::Integer=1,
    allowed_devices=nothing,
    memory_fraction::Real=0.75,
    kwargs...,
)
    err = Ref{Cstring}(C_NULL)
    ids = allowed_devices === nothing ? Int64[] : collect(Int64, allowed_devices)
    client = ccall(
        sym(:MakeGPUClient),
        Ptr{Cvoid},
        (Cint, Cint, Ptr{Int64}, Int64, Cdouble, UInt8, Cstring, Ptr{Cstring}, Ptr{Cvoid}),
        node_id, num_nodes, isempty(ids) ? C_NULL : pointer(ids), length(ids),
        memory_fraction, false, "cuda", err, C_NULL,
    )
    client == C_NULL && error(unsafe_string(err[]))
    return PJRT.Client(client)
end

# XLA.compile for this backend.  The reference calls
# ClientCompileWithProto(client, mod, opts, n) (src/xla/PJRT/LoadedExecutable.jl:62-83);
# this library does not link MLIR, so the optimised module crosses as text.
function XLA.compile(
    client::PJRT.Client,
    mod::MLIR.IR.Module;
    compile_options,
    num_parameters::Int64,
    num_outputs::Int64,
    is_sharded::Bool,
    num_replicas::Int64,
    num_partitions::Int64,
    kwargs...,
)
    text = string(mod)
    exec = ccall(
        sym(:ClientCompileText),
        Ptr{Cvoid},
        (Ptr{Cvoid}, Cstring, Csize_t, Ptr{UInt8}, Csize_t),
        client.client, text, sizeof(text), C_NULL, 0,
    )
    return PJRT.LoadedExecutable(
        exec, num_outputs, num_parameters, is_sharded, num_replicas, num_partitions
    )
end

# What Codegen asserts against the inputs (src/compiler/Codegen.jl:797-809): the tensor
# dimension split over the 1-D mesh, or -1 for a replicated value.
function parameter_sharded_dims(exec::PJRT.LoadedExecutable)
    return [
        ccall(sym(:RxExecutableParameterShardedDim), Cint, (Ptr{Cvoid}, Cint), exec.exec, i - 1)
        for i in 1:(exec.num_parameters)
    ]
end

function result_sharded_dims(exec::PJRT.LoadedExecutable)
    return [
        ccall(sym(:RxExecutableResultShardedDim), Cint, (Ptr{Cvoid}, Cint), exec.exec, i - 1)
        for i in 1:(exec.num_outputs)
    ]
end

# The launch plan (fusion groups and kernels) as JSON: the counterpart of dumping the
# compiled HLO.
function describe(exec::PJRT.LoadedExecutable)
    p = ccall(sym(:RxExecutableDescribe), Cstring, (Ptr{Cvoid},), exec.exec)
    s = unsafe_string(p)
    Libc.free(p)
    return s
end

end # module
