# B200Backend.jl -- puts librx_b200.so behind Reactant.jl's PJRT wrapper structs.
#
# Written against Reactant.jl v0.2.280.  Julia is not installed where the engine is built, so this file has not
# been executed there.  Every entry point it binds is exercised from Python through the same C ABI in the test
# suite, and a test parses the `rx(...)` table below and checks every name and arity against include/rx_b200.h.
#
# How the binding works
# ---------------------
# Reactant's wrappers (src/xla/PJRT/{Client,Device,Buffer,Future,LoadedExecutable}.jl) hold one raw pointer each
# and reach the runtime through the stubs of `MLIR.API` (src/mlir/libMLIR_h.jl, e.g. :15303-15305 ClientNumDevices,
# :15453 ArrayFromHostBuffer), which are plain `@ccall`s into libReactantExtra.  This module adds, for every stub
# of the client / device / buffer / future / executable groups, a method of the same name and arity that asks the
# library whether the handle is one of its own (`RxOwns`) and, if so, makes the same call into librx_b200.so;
# any other handle (the XLA CPU client lives in the same session) goes to the stub as it was when this module was
# loaded (`Base.invoke_in_world`).  The wrapper structs, `ConcretePJRTArray`, the generated thunks and the
# finalizers are used unchanged.
module B200Backend

using Reactant: Reactant, XLA, MLIR
using Reactant.XLA: PJRT
using Libdl

const lib = Ref{Ptr{Cvoid}}(C_NULL)
# the world in which `MLIR.API.*` still are Reactant's own stubs
const stock_world = Ref{UInt}(0)

sym(name::Symbol) = Libdl.dlsym(lib[], name)
owns(p) = p != C_NULL && ccall(sym(:RxOwns), UInt8, (Ptr{Cvoid},), p) != 0

# ---- the entry points, with the argument and result types of src/mlir/libMLIR_h.jl ----------------------------
# rx(name, result type, (argument types...), index of the argument whose ownership routes the call)
const TABLE = Any[]
rx(name, ret, args, handle=1) = push!(TABLE, (name, ret, args, handle))

const P = Ptr{Cvoid}
rx(:FreeClient, Cvoid, (P,))
rx(:ClientNumDevices, Cint, (P,))
rx(:ClientNumAddressableDevices, Cint, (P,))
rx(:ClientProcessIndex, Cint, (P,))
rx(:ClientGetDevice, P, (P, Cint))
rx(:ClientGetAddressableDevice, P, (P, Cint))
rx(:ClientGetDevices, Cvoid, (P, Ptr{P}))
rx(:ClientGetAddressableDevices, Cvoid, (P, Ptr{P}))
rx(:ClientGetPlatformName, Cstring, (P,))
rx(:DeviceToClient, P, (P,))
rx(:PjRtDeviceGetLocalDeviceId, Int64, (P,))
rx(:PjRtDeviceGetGlobalDeviceId, Int64, (P,))
rx(:PjRtDeviceGetLocalHardwareId, Int64, (P,))
rx(:DeviceGetKind, Cstring, (P,))
rx(:pjrt_device_is_addressable, Bool, (P,))
rx(:PjRtDeviceGetAllocatorStats, Cvoid, (P, P))
rx(:ArrayFromHostBuffer, P, (P, P, UInt64, Csize_t, Ptr{Int64}, P))
rx(:UninitPJRTBuffer, P, (P, P, UInt64, UInt64, Ptr{UInt64}))
rx(:PjRtBufferFree, Cvoid, (P,))
rx(:BufferShape, Ptr{Int64}, (P,))
rx(:BufferNDimensions, Int64, (P,))
rx(:BufferPrimitiveType, Cint, (P,))
rx(:BufferToDevice, P, (P,))
rx(:BufferToClient, P, (P,))
rx(:BufferOnCPU, UInt8, (P,))
rx(:BufferToHost, Cvoid, (P, P))
rx(:UnsafeBufferPointer, P, (P,))
rx(:CopyBufferToDevice, P, (P, P))
rx(:CopyToBuffer, Cvoid, (P, P, P, Csize_t, Csize_t, Ptr{P}), 2)
rx(:CopyFromBuffer, Cvoid, (P, P, P, Csize_t, Csize_t, Ptr{P}), 2)
rx(:FreeFuture, Cvoid, (P,))
rx(:FutureIsReady, UInt8, (P,))
rx(:FutureAwait, Cvoid, (P,))
rx(:ExecutableFree, Cvoid, (P,))
rx(:PjRtLoadedExecutableGetClient, P, (P,))
rx(:PjRtLoadedExecutableNumReplicas, Cint, (P,))
rx(:PjRtLoadedExecutableNumPartitions, Cint, (P,))
rx(:PjRtLoadedExecutableGetParameterShardings, Cvoid, (P, Ptr{P}, Int32))
rx(:PjRtLoadedExecutableGetOuputShardings, Cvoid, (P, Ptr{P}, Int32))
rx(:PjRtLoadedExecutableGetHloModules, Cvoid, (P, Ptr{P}, Ptr{Int32}))
rx(:XLAExecuteSharded, Cvoid, (P, Cint, Ptr{P}, P, Ptr{UInt8}, Cint, Ptr{P}, Ptr{UInt8}, Ptr{P}))
rx(:XLAExecute, Cvoid, (P, Cint, Ptr{P}, Ptr{UInt8}, Cint, Ptr{P}, Ptr{UInt8}, Ptr{P}))
# the OpSharding objects the two sharding getters hand out, and their accessors (src/xla/Sharding.jl:20-120)
rx(:free_op_sharding, Cvoid, (P,))
rx(:op_sharding_to_op_sharding_type, Int32, (P,))
rx(:op_sharding_to_shard_group_type, Int32, (P,))
rx(:op_sharding_to_shard_group_id, Int32, (P,))
rx(:op_sharding_is_shard_group, Bool, (P,))
rx(:op_sharding_replicate_on_last_tile_dim, Bool, (P,))
rx(:op_sharding_has_last_tile_dims, Bool, (P,))
rx(:op_sharding_last_tile_dims_size, Int32, (P,))
rx(:op_sharding_last_tile_dims, Cvoid, (P, Ptr{Int32}))
rx(:op_sharding_has_iota_reshape_dims, Bool, (P,))
rx(:op_sharding_iota_reshape_dims_size, Int32, (P,))
rx(:op_sharding_iota_reshape_dims, Cvoid, (P, Ptr{Int32}))
rx(:op_sharding_has_iota_transpose_perm, Bool, (P,))
rx(:op_sharding_iota_transpose_perm_size, Int32, (P,))
rx(:op_sharding_iota_transpose_perm, Cvoid, (P, Ptr{Int32}))
rx(:op_sharding_has_tile_assignment_dimensions, Bool, (P,))
rx(:op_sharding_tile_assignment_dimensions_size, Int32, (P,))
rx(:op_sharding_tile_assignment_dimensions, Cvoid, (P, Ptr{Int32}))
rx(:op_sharding_has_tile_assignment_devices, Bool, (P,))
rx(:op_sharding_tile_assignment_devices_size, Int32, (P,))
rx(:op_sharding_tile_assignment_devices, Cvoid, (P, Ptr{Int32}))

# The OpSharding handles are plain heap objects of this library, not in the ownership table: the binding keeps
# its own record of the ones it handed to Julia.
const OP_SHARDINGS = Set{Ptr{Cvoid}}()
const OP_SHARDINGS_LOCK = ReentrantLock()

handle_is_ours(name::Symbol, h) =
    if startswith(String(name), "op_sharding_") || name === :free_op_sharding
        @lock OP_SHARDINGS_LOCK (h in OP_SHARDINGS)
    else
        owns(h)
    end

# One method per table row, added to MLIR.API.  Arguments arrive as whatever the wrapper passes (raw pointers,
# Refs, arrays); `Base.cconvert` / `unsafe_convert` bring them to the C types exactly as `@ccall` would.
function install_overrides()
    for (name, ret, args, handle) in TABLE
        n = length(args)
        vars = [Symbol(:a, i) for i in 1:n]
        argtypes = Expr(:tuple, args...)
        @eval MLIR.API function $name($(vars...))
            h = Base.unsafe_convert($(args[handle]), Base.cconvert($(args[handle]), $(vars[handle])))
            if $(handle_is_ours)($(QuoteNode(name)), reinterpret(Ptr{Cvoid}, h))
                r = ccall($(sym)($(QuoteNode(name))), $ret, $argtypes, $(vars...))
                $(after_call)($(QuoteNode(name)), $(vars...))
                return r
            end
            return Base.invoke_in_world($(stock_world)[], $name, $(vars...))
        end
    end
    return nothing
end

# bookkeeping for the OpSharding objects
function after_call(name::Symbol, args...)
    if name === :PjRtLoadedExecutableGetParameterShardings || name === :PjRtLoadedExecutableGetOuputShardings
        out = Base.unsafe_convert(Ptr{Ptr{Cvoid}}, Base.cconvert(Ptr{Ptr{Cvoid}}, args[2]))
        @lock OP_SHARDINGS_LOCK for i in 1:Int(args[3])
            push!(OP_SHARDINGS, unsafe_load(out, i))
        end
    elseif name === :free_op_sharding
        @lock OP_SHARDINGS_LOCK delete!(OP_SHARDINGS, reinterpret(Ptr{Cvoid}, args[1]))
    end
    return nothing
end

# ---- device properties: answered for every CUDA device, whichever client asks (src/xla/Device.jl:43-60) -------
function install_device_queries()
    @eval MLIR.API function ReactantCudaDeviceGetProperties(jlprops, device_id)
        return ccall($(sym)(:ReactantCudaDeviceGetProperties), Cvoid, (Ptr{Cvoid}, Int32), jlprops, device_id)
    end
    @eval MLIR.API function ReactantCudaDriverGetVersion()
        return ccall($(sym)(:ReactantCudaDriverGetVersion), Int32, ())
    end
    return nothing
end

# ---- client: MakeGPUClient with the reference signature (deps/ReactantExtra/API.cpp:528-582) ------------------
# Same keyword arguments as the stock factory (src/accelerators/GPU.jl:7-37), which Reactant passes from
# src/xla/XLA.jl:271-308: node_id, num_nodes, distributed_runtime_client, allowed_devices
# (REACTANT_VISIBLE_GPU_DEVICES, src/xla/XLA.jl:230-233).
function make_pjrt_client(;
    node_id::Integer=0,
    num_nodes::Integer=1,
    distributed_runtime_client=nothing,
    allowed_devices::Union{Nothing,Vector{Int}}=nothing,
)
    err = Ref{Cstring}(C_NULL)
    ids = allowed_devices === nothing ? Int64[] : collect(Int64, allowed_devices)
    client = GC.@preserve ids err ccall(
        sym(:MakeGPUClient),
        Ptr{Cvoid},
        (Cint, Cint, Ptr{Int64}, Int64, Cdouble, UInt8, Cstring, Ptr{Cstring}, Ptr{Cvoid}),
        node_id, num_nodes, isempty(ids) ? C_NULL : pointer(ids), length(ids),
        XLA.XLA_REACTANT_GPU_MEM_FRACTION[], XLA.XLA_REACTANT_GPU_PREALLOCATE[], "gpu", err, C_NULL,
    )
    client == C_NULL && throw(AssertionError(unsafe_string(err[])))
    return PJRT.Client(client)  # the wrapper's own calls (ClientNumDevices, ...) now route here by ownership
end

# ---- compile ------------------------------------------------------------------------------------------------
# The reference calls ClientCompileWithProto(client, mod, opts, n) (src/xla/PJRT/LoadedExecutable.jl:62-83).  This
# library does not link MLIR, so for one of its own clients the optimised module crosses as text
# (ClientCompileText); any other client takes Reactant's own method.
function compile_text(client::PJRT.Client, mod::MLIR.IR.Module; num_parameters, num_outputs, is_sharded, num_replicas, num_partitions)
    text = string(mod)
    exec = GC.@preserve client text ccall(
        sym(:ClientCompileText),
        Ptr{Cvoid},
        (Ptr{Cvoid}, Cstring, Csize_t, Ptr{UInt8}, Csize_t),
        client.client, text, sizeof(text), C_NULL, 0,
    )
    exec == C_NULL && error(unsafe_string(ccall(sym(:RxLastError), Cstring, ())))
    return PJRT.LoadedExecutable(exec, num_outputs, num_parameters, is_sharded, num_replicas, num_partitions)
end

function install_compile()
    @eval function XLA.compile(
        client::PJRT.Client,
        mod::MLIR.IR.Module;
        compile_options,
        num_parameters::Int64,
        num_outputs::Int64,
        is_sharded::Bool,
        num_replicas::Int64,
        num_partitions::Int64,
    )
        if $(owns)(client.client)
            return $(compile_text)(client, mod; num_parameters, num_outputs, is_sharded, num_replicas, num_partitions)
        end
        return Base.invoke_in_world(
            $(stock_world)[], XLA.compile, client, mod;
            compile_options, num_parameters, num_outputs, is_sharded, num_replicas, num_partitions,
        )
    end
    return nothing
end

# ---- execute --------------------------------------------------------------------------------------------------
# Multi-device thunks call MLIR.API.XLAExecute (src/xla/PJRT/LoadedExecutable.jl:292-329), routed by the table
# above.  Single-device thunks call the symbol `XLAExecuteSharded` straight from generated LLVM IR, resolved in
# Julia's JIT dylib to libReactantExtra's function (src/xla/XLA.jl:244-258), which the table cannot see.  For those
# the generated method is replaced by the form Reactant itself uses while precompiling (plain call through
# MLIR.API.XLAExecuteSharded, :225-246), and the library is given the stock functions so that its own exported
# symbols, should anything still bind to them by name, pass foreign executables on.
function install_execute()
    stock = Reactant.Reactant_jll.libReactantExtra_handle
    ccall(sym(:RxSetForeignExecute), Cvoid, (Ptr{Cvoid}, Ptr{Cvoid}), Libdl.dlsym(stock, :XLAExecuteSharded), Libdl.dlsym(stock, :XLAExecute))
    @eval function XLA.execute_sharded(
        exec::PJRT.LoadedExecutable,
        device::PJRT.Device,
        inputs::NTuple{N,Ptr{Cvoid}},
        donated_args::NTuple{N,UInt8},
        ::Val{n_outs},
    ) where {N,n_outs}
        if !$(owns)(exec.exec)
            return Base.invoke_in_world($(stock_world)[], XLA.execute_sharded, exec, device, inputs, donated_args, Val(n_outs))
        end
        outputs_p = Ref{NTuple{n_outs,Ptr{Cvoid}}}()
        futures_res = Ref{NTuple{n_outs,Ptr{Cvoid}}}()
        futures = Ref{UInt8}(0)
        GC.@preserve exec device begin
            MLIR.API.XLAExecuteSharded(
                exec.exec, N, Base.RefValue(inputs), device.device, Base.RefValue(donated_args),
                n_outs, outputs_p, futures, futures_res,
            )
        end
        outputs, future_res, future = outputs_p[], futures_res[], futures[] != 0
        return ntuple(Val(n_outs)) do i
            (PJRT.AsyncBuffer(PJRT.Buffer(outputs[i]), future ? PJRT.Future(future_res[i]) : nothing),)
        end
    end
    return nothing
end

function __init__()
    lib[] = Libdl.dlopen(get(ENV, "RX_B200_LIB", "librx_b200.so"))
    # Runtime failures are reported through the slot Reactant installs its throwing callback in
    # (src/xla/XLA.jl:203-204, deps/ReactantExtra/API.cpp:262).
    unsafe_store!(Ptr{Ptr{Cvoid}}(sym(:ReactantThrowError)), @cfunction(XLA.reactant_err, Cvoid, (Cstring,)))
    stock_world[] = Base.get_world_counter()
    install_overrides()
    install_device_queries()
    install_compile()
    install_execute()
    # `register_backend(platform_name; priority, pjrt_initialize_function, ...)` (src/accelerators/Registration.jl:24-54)
    # refuses a name that is already taken, and the stock GPU module registers "cuda" at priority 500 in its own
    # __init__ (src/accelerators/GPU.jl:71-92).  Its entry is replaced in place, so that "cuda" -- what
    # `Reactant.set_default_backend("gpu")` looks up first (src/xla/XLA.jl:131-138) and what the compiler maps to
    # its GPU pipeline (src/compiler/Compiler.jl:61-65) -- is served by this engine; without a stock entry a
    # fresh one is added at the same priority.
    R = Reactant.Accelerators.Registration
    @lock R.BackendRegistrationLock begin
        filter!(b -> b.platform_name != "cuda", R.RegisteredBackends)
    end
    R.register_backend("cuda"; priority=500, pjrt_initialize_function=make_pjrt_client)
    return nothing
end

# The launch plan (fusion groups and kernels) as JSON: the counterpart of dumping the compiled HLO.
function describe(exec::PJRT.LoadedExecutable)
    p = ccall(sym(:RxExecutableDescribe), Cstring, (Ptr{Cvoid},), exec.exec)
    s = unsafe_string(p)
    Libc.free(p)
    return s
end

end # module
