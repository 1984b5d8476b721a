(* b200_backend.ml — OCaml half of the Blackwell backend: an implementation of
   [Backend_impl.Lowered_backend] (arrayjit/lib/backend_impl.ml:334-367) that forwards every member
   to libb200.so (include/b200.h) through ctypes.

   STATUS: source only.  No OCaml toolchain exists in the environment this backend was built in, so
   this file has never been compiled; it documents the binding precisely enough to finish on a
   machine with OCaml >= 5.3.  The C ABI underneath is exercised by the Python ctypes mirror
   (ocannl_b200/backend.py), which follows the same call sequence.

   It is modelled on arrayjit/lib/cuda_backend.ml (device/stream/event/pool handling) with the
   cudajit calls replaced by the C ABI, and on arrayjit/lib/cc_backend.ml:378-443 for ctypes use. *)

open Base
module Tn = Tnode
module Lazy = Utils.Lazy
open Ctypes
open Foreign

let lib = Dl.dlopen ~filename:"libb200.so" ~flags:[ Dl.RTLD_NOW; Dl.RTLD_GLOBAL ]
let vp = ptr void
let last_error = foreign ~from:lib "b200_last_error" (void @-> returning string)

let check rc =
  if rc = 0 then ()
  else
    let msg = last_error () in
    if rc = -5 then raise (Utils.User_error msg)
    else if rc = -1 then invalid_arg msg
    else failwith (Printf.sprintf "b200 (%d): %s" rc msg)

let c_init = foreign ~from:lib "b200_init" (void @-> returning int)
let c_num_devices = foreign ~from:lib "b200_num_devices" (ptr int @-> returning int)
let c_device_open = foreign ~from:lib "b200_device_open" (int @-> ptr vp @-> returning int)
let c_device_props = foreign ~from:lib "b200_device_props" (vp @-> ptr char @-> size_t @-> returning int)
let c_pool_alloc = foreign ~from:lib "b200_pool_alloc" (vp @-> int @-> size_t @-> size_t @-> returning int)
let c_pool_free = foreign ~from:lib "b200_pool_free" (vp @-> int @-> returning int)
let c_pool_memset0 = foreign ~from:lib "b200_pool_memset0" (vp @-> int @-> size_t @-> size_t @-> returning int)
let c_h2d = foreign ~from:lib "b200_h2d" (vp @-> int @-> size_t @-> vp @-> size_t @-> returning int)
let c_d2h = foreign ~from:lib "b200_d2h" (vp @-> int @-> size_t @-> vp @-> size_t @-> returning int)
(* extension: from_host copies on a second stream, ordered per pool (include/b200.h) *)
let c_set_async_uploads = foreign ~from:lib "b200_set_async_uploads" (vp @-> int @-> returning int)

let c_d2d =
  foreign ~from:lib "b200_d2d" (vp @-> int @-> size_t @-> vp @-> int @-> size_t @-> size_t @-> returning int)

let c_merge_copy = foreign ~from:lib "b200_merge_copy" (vp @-> vp @-> int @-> size_t @-> size_t @-> returning int)
let c_event_record = foreign ~from:lib "b200_event_record" (vp @-> ptr vp @-> returning int)
let c_event_query = foreign ~from:lib "b200_event_query" (vp @-> ptr int @-> returning int)
let c_event_sync = foreign ~from:lib "b200_event_sync" (vp @-> returning int)
let c_event_free = foreign ~from:lib "b200_event_free" (vp @-> returning int)
let c_stream_wait = foreign ~from:lib "b200_stream_wait" (vp @-> vp @-> returning int)
let c_await = foreign ~from:lib "b200_await" (vp @-> returning int)
let c_is_idle = foreign ~from:lib "b200_is_idle" (vp @-> ptr int @-> returning int)
let c_used_memory = foreign ~from:lib "b200_used_memory" (vp @-> ptr size_t @-> returning int)

let c_compile =
  foreign ~from:lib "b200_compile" (string @-> string @-> size_t @-> string_opt @-> ptr vp @-> returning int)

type binding
let binding : binding structure typ = structure "b200_binding"
let b_tn = field binding "tn_id" int32_t
let b_pool = field binding "pool_id" int32_t
let b_off = field binding "offset" uint64_t
let () = seal binding

(* bindings need only be aligned to the element size, as Raise_backend.allocate_delta hands them out
   (arrayjit/lib/backends.ml:529-614): the library re-plans stages that wanted more *)
let c_link = foreign ~from:lib "b200_link" (vp @-> vp @-> ptr binding @-> int @-> ptr vp @-> returning int)
let c_routine_info = foreign ~from:lib "b200_routine_info" (vp @-> ptr char @-> size_t @-> returning int)

(* data-parallel exchange (used by parallel_b200.ml) *)
let c_comm_unique_id = foreign ~from:lib "b200_comm_unique_id" (ptr char @-> returning int)
let c_comm_init_rank = foreign ~from:lib "b200_comm_init_rank" (vp @-> int @-> int @-> ptr char @-> ptr vp @-> returning int)
let c_allreduce = foreign ~from:lib "b200_allreduce" (vp @-> int @-> size_t @-> size_t @-> int @-> int @-> returning int)

let c_overlap_allreduce =
  foreign ~from:lib "b200_routine_overlap_allreduce"
    (vp @-> vp @-> int @-> ptr int @-> ptr size_t @-> ptr size_t @-> int @-> int @-> returning int)

let c_comm_init_all = foreign ~from:lib "b200_comm_init_all" (int @-> ptr vp @-> ptr vp @-> returning int)

let c_allreduce_all =
  foreign ~from:lib "b200_allreduce_all" (int @-> ptr vp @-> ptr int @-> ptr size_t @-> size_t @-> int @-> int @-> returning int)

let c_comm_set_timeout = foreign ~from:lib "b200_comm_set_timeout" (vp @-> llong @-> returning int)
let c_comm_free = foreign ~from:lib "b200_comm_free" (vp @-> returning int)
let c_launch = foreign ~from:lib "b200_launch" (vp @-> ptr int64_t @-> int @-> returning int)
let c_use_graph = foreign ~from:lib "b200_routine_use_graph" (vp @-> int @-> returning int)

(* ---------------------------------------------------------------- b200ir serialiser
   Writes the wire format documented in ocannl_b200/low_level.py.  Forces [tn.prec] / [tn.dims]
   (safe at compile time: [C_syntax] forces them too, arrayjit/lib/c_syntax.ml:482-483), writes each
   traced node once with the memory class [C_syntax.compile_proc] derives
   (arrayjit/lib/c_syntax.ml:1028-1043), then the statement tree. *)
module Ser = struct
  open Low_level

  let buf_add = Buffer.add_string
  let hexfloat c =
    if Float.is_nan c then "nan"
    else if Float.(c = infinity) then "inf"
    else if Float.(c = neg_infinity) then "-inf"
    else Printf.sprintf "%h" c

  let idx = function
    | Indexing.Fixed_idx i -> Int.to_string i
    | Iterator s -> Indexing.symbol_ident s
    | Affine { symbols; offset } ->
        "(affine " ^ Int.to_string offset ^ " "
        ^ String.concat ~sep:" "
            (List.map symbols ~f:(fun (c, s) -> Printf.sprintf "(%d %s)" c (Indexing.symbol_ident s)))
        ^ ")"
    | Sub_axis -> "sub_axis"
    | Concat _ -> invalid_arg "b200: Concat indices are eliminated during lowering"

  let idcs a = "(" ^ String.concat_array ~sep:" " (Array.map a ~f:idx) ^ ")"
  let prec p = Ops.prec_string p

  let binop = function
    | Ops.Arg1 -> "arg1" | Arg2 -> "arg2" | Add -> "add" | Sub -> "sub" | Mul -> "mul" | Div -> "div"
    | ToPowOf -> "pow" | Relu_gate -> "relu_gate" | Satur01_gate -> "sat01_gate" | Cmplt -> "lt"
    | Cmpeq -> "eq" | Cmpne -> "ne" | Or -> "or" | And -> "and" | Mod -> "mod" | Max -> "max" | Min -> "min"
    | Threefry4x32_crypto -> "threefry4x32_crypto" | Threefry4x32_light -> "threefry4x32_light"

  let unop = function
    | Ops.Identity -> "id" | Relu -> "relu" | Satur01 -> "sat01" | Exp -> "exp" | Log -> "log" | Exp2 -> "exp2"
    | Log2 -> "log2" | Sin -> "sin" | Cos -> "cos" | Sqrt -> "sqrt" | Recip -> "recip"
    | Recip_sqrt -> "recip_sqrt" | Neg -> "neg" | Trunc -> "trunc" | Tanh_approx -> "tanh" | Not -> "not"
    | Uint4x32_to_prec_uniform1 -> "uint4x32_to_prec_uniform1"

  let ternop = function Ops.Where -> "where" | FMA -> "fma" | Mul3 -> "mul3"

  let rec stmt b = function
    | Noop -> buf_add b "(noop)"
    | Comment s -> buf_add b (Printf.sprintf "(comment %S)" s)
    | Staged_compilation _ -> invalid_arg "b200: Staged_compilation cannot cross the backend boundary"
    | Seq (c1, c2) -> buf_add b "(seq "; stmt b c1; buf_add b " "; stmt b c2; buf_add b ")"
    | For_loop { index; from_; to_; body; _ } ->
        buf_add b (Printf.sprintf "(for %s %d %d " (Indexing.symbol_ident index) from_ to_);
        stmt b body; buf_add b ")"
    | Zero_out tn -> buf_add b (Printf.sprintf "(zero_out %d)" tn.Tn.id)
    | Set { tn; idcs = i; llsc; _ } ->
        buf_add b (Printf.sprintf "(set %d %s " tn.Tn.id (idcs i)); scalar b llsc; buf_add b ")"
    | Set_from_vec { tn; idcs = i; length; vec_unop = Ops.Uint4x32_to_prec_uniform; arg; _ } ->
        (* the only vector operation (arrayjit/lib/ops.ml:452): `length` results of the uniform
           conversion of one uint4x32 value go to consecutive elements starting at idcs *)
        buf_add b (Printf.sprintf "(set_from_vec %d %s %d uint4x32_to_prec_uniform " tn.Tn.id (idcs i) length);
        arg_ b arg; buf_add b ")"
    | Set_local ({ scope_id; tn }, v) ->
        buf_add b (Printf.sprintf "(set_local %d %d " scope_id tn.Tn.id); scalar b v; buf_add b ")"
    | Declare_local { id = { scope_id; tn }; needs_init } ->
        buf_add b (Printf.sprintf "(declare_local %d %d %d)" scope_id tn.Tn.id (Bool.to_int needs_init))

  and arg b (s, p) = buf_add b "("; scalar b s; buf_add b (" " ^ prec p ^ ")")
  and arg_ b a = arg b a

  and scalar b = function
    | Local_scope { id = { scope_id; tn }; body; orig_indices } ->
        buf_add b (Printf.sprintf "(scope %d %d " scope_id tn.Tn.id); stmt b body;
        buf_add b (" " ^ idcs orig_indices ^ ")")
    | Get_local { scope_id; tn } -> buf_add b (Printf.sprintf "(get_local %d %d)" scope_id tn.Tn.id)
    | Get (tn, i) -> buf_add b (Printf.sprintf "(get %d %s)" tn.Tn.id (idcs i))
    | Get_merge_buffer (tn, i) -> buf_add b (Printf.sprintf "(get_merge %d %s)" tn.Tn.id (idcs i))
    | Get_dynamic { tn; idcs = i; dyn_axis; dyn_value } ->
        buf_add b (Printf.sprintf "(get_dyn %d %s %d " tn.Tn.id (idcs i) dyn_axis); arg b dyn_value; buf_add b ")"
    | Ternop (op, a1, a2, a3) ->
        buf_add b ("(tern " ^ ternop op ^ " "); arg b a1; buf_add b " "; arg b a2; buf_add b " "; arg b a3; buf_add b ")"
    | Binop (op, a1, a2) -> buf_add b ("(bin " ^ binop op ^ " "); arg b a1; buf_add b " "; arg b a2; buf_add b ")"
    | Unop (op, a) -> buf_add b ("(un " ^ unop op ^ " "); arg b a; buf_add b ")"
    | Constant c -> buf_add b ("(const " ^ hexfloat c ^ ")")
    | Constant_bits i -> buf_add b (Printf.sprintf "(const_bits %Ld)" i)
    | Embed_index i -> buf_add b ("(idx " ^ idx i ^ ")")

  let optimized ~name ~(bindings : Indexing.unit_bindings) ~in_ctx
      ({ traced_store; llc; merge_node; _ } : Low_level.optimized) =
    let b = Buffer.create 4096 in
    let ident = Low_level.get_ident_within_code [| llc |] in
    buf_add b (Printf.sprintf "(b200ir 1 (name %s)\n (tnodes\n" name);
    Hashtbl.iteri traced_store ~f:(fun ~key:tn ~data:node ->
        let mode =
          if Tn.is_virtual_force tn 3341 then "virtual"
          else if in_ctx tn then "ctx"
          else if Tn.is_materialized_force tn 3351 then "global"
          else "local"
        in
        buf_add b
          (Printf.sprintf "  (tn %d %s %s (%s) %s%s%s)\n" tn.Tn.id (ident tn) (prec (Lazy.force tn.prec))
             (String.concat_array ~sep:" " (Array.map (Lazy.force tn.dims) ~f:Int.to_string))
             mode
             (if node.Low_level.zero_initialized_by_code then " zero_init" else "")
             (if node.read_only then " read_only" else "")));
    buf_add b " )\n (static";
    List.iter (Indexing.bound_symbols bindings) ~f:(fun { Indexing.static_symbol; static_range } ->
        buf_add b
          (Printf.sprintf " (%s %s)" (Indexing.symbol_ident static_symbol)
             (Option.value_map static_range ~default:"none" ~f:Int.to_string)));
    buf_add b ")\n (merge ";
    buf_add b (Option.value_map merge_node ~default:"none" ~f:(fun tn -> Int.to_string tn.Tn.id));
    buf_add b ")\n (body ";
    stmt b llc;
    buf_add b "))\n";
    Buffer.contents b
end

(* ---------------------------------------------------------------- the backend *)
module Fresh () : Backend_impl.Lowered_backend = struct
  include Backend_impl.No_device_buffer_and_copying ()  (* host-side defaults; see cuda_backend.ml *)

  type dev = { handle : unit ptr; ordinal : int }
  type runner = unit  (* the single stream lives inside the library *)
  type event = unit ptr

  type code = { handle : unit ptr; name : string; params : Tn.t list; statics : Indexing.static_symbol list }
  [@@deriving sexp_of]

  type code_batch = code option array [@@deriving sexp_of]

  let () = check (c_init ())
  let name = "b200"

  let num_devices () =
    let n = allocate int 0 in
    check (c_num_devices n);
    !@n

  let devices = Hashtbl.create (module Int)

  let get_device ~ordinal =
    Hashtbl.find_or_add devices ordinal ~default:(fun () ->
        let h = allocate vp null in
        check (c_device_open ordinal h);
        make_device { handle = !@h; ordinal } () ~ordinal)

  (* Slab_alloc (backend_intf.ml:22-37) *)
  let alloc_pool ?mode:_ device ~pool_id ~size_in_bytes ~alignment =
    check (c_pool_alloc device.dev.handle pool_id (Unsigned.Size_t.of_int size_in_bytes) (Unsigned.Size_t.of_int alignment))

  let free_pool device ~pool_id = check (c_pool_free device.dev.handle pool_id)

  let memset_zero device ~pool_id ~offset ~size_in_bytes =
    check (c_pool_memset0 device.dev.handle pool_id (Unsigned.Size_t.of_int offset) (Unsigned.Size_t.of_int size_in_bytes))

  (* copies (backend_impl.ml:292-315) *)
  let from_host ~dst ~dst_loc:{ Backend_intf.pool_id; offset } nd =
    let f src = check (c_h2d dst.device.dev.handle pool_id (Unsigned.Size_t.of_int offset)
                         (to_voidp (bigarray_start genarray src)) (Unsigned.Size_t.of_int (Ndarray.size_in_bytes nd))) in
    Ndarray.apply { f } nd

  let to_host ~src ~src_loc:{ Backend_intf.pool_id; offset } nd =
    let f dst = check (c_d2h src.device.dev.handle pool_id (Unsigned.Size_t.of_int offset)
                         (to_voidp (bigarray_start genarray dst)) (Unsigned.Size_t.of_int (Ndarray.size_in_bytes nd))) in
    Ndarray.apply { f } nd

  let device_to_device tn ~into_merge_buffer ~dst_loc ~dst ~src_loc ~src =
    let bytes = Unsigned.Size_t.of_int (Lazy.force tn.Tn.size_in_bytes) in
    let s_off = Unsigned.Size_t.of_int src_loc.Backend_intf.offset in
    match (into_merge_buffer, dst_loc) with
    | Backend_intf.No, None -> invalid_arg "b200: device_to_device: missing dst_loc"
    | No, Some d ->
        check (c_d2d dst.device.dev.handle d.pool_id (Unsigned.Size_t.of_int d.offset) src.device.dev.handle
                 src_loc.pool_id s_off bytes)
    | Copy, _ ->
        check (c_merge_copy dst.device.dev.handle src.device.dev.handle src_loc.pool_id s_off bytes);
        dst.device.merge_buffer := Some { Backend_intf.pool_id = 0; offset = 0 }
    | Streaming_for _, _ -> failwith "b200: streaming merge buffers are not supported"

  (* events and stream (backend_intf.ml:97-126) *)
  let all_work device =
    let e = allocate vp null in
    check (c_event_record device.dev.handle e);
    let ev = !@e in
    Stdlib.Gc.finalise (fun ev -> ignore (c_event_free ev)) ev;
    ev

  let is_done ev = let d = allocate int 0 in check (c_event_query ev d); !@d <> 0
  let sync ev = check (c_event_sync ev)
  let will_wait_for context ev = check (c_stream_wait context.device.dev.handle ev)
  let await device = check (c_await device.dev.handle)
  let is_idle device = let d = allocate int 0 in check (c_is_idle device.dev.handle d); !@d <> 0

  let get_used_memory device =
    let n = allocate size_t Unsigned.Size_t.zero in
    check (c_used_memory device.dev.handle n);
    Unsigned.Size_t.to_int !@n

  (* Compile options of the library ("key=0|1 ..."), from ocannl_config entries b200_<key> (as the cc
     backend reads cc_backend_* there, utils.ml:242); absent entries keep the library's defaults. *)
  let compile_options =
    lazy
      (let keys = [ "gemm"; "attn"; "tf32"; "splitk"; "coop"; "fuse"; "pairs"; "bounds" ] in
       let set =
         List.filter_map keys ~f:(fun k ->
             match Utils.get_global_arg ~default:"" ~arg_name:("b200_" ^ k) with
             | "" -> None
             | v -> Some (k ^ "=" ^ if String.(v = "true" || v = "1") then "1" else "0"))
       in
       let set = if Utils.settings.large_models then "large_models=1" :: set else set in
       if List.is_empty set then None else Some (String.concat ~sep:" " set))

  (* compile / link (backend_impl.ml:334-367) *)
  let compile ~name bindings (lowered : Low_level.optimized) =
    let params =
      Hashtbl.keys lowered.traced_store
      |> List.filter ~f:(fun tn -> Tn.is_in_context_force tn 3361 || Tn.is_materialized_force tn 3362)
    in
    let text = Ser.optimized ~name ~bindings ~in_ctx:(fun tn -> Tn.is_in_context_force tn 3363) lowered in
    let h = allocate vp null in
    check (c_compile name text (Unsigned.Size_t.of_int (String.length text)) (Lazy.force compile_options) h);
    { handle = !@h; name; params; statics = Indexing.bound_symbols bindings }

  let compile_batch ~names bindings lowereds =
    Array.mapi lowereds ~f:(fun i ->
        Option.map ~f:(fun l -> compile ~name:(Option.value names.(i) ~default:("routine" ^ Int.to_string i)) bindings l))

  let link prior_context (code : code) (ctx_buffers : Backend_intf.buffer_loc Map.M(Tn).t) =
    let n = List.length code.params in
    let arr = CArray.make binding n in
    List.iteri code.params ~f:(fun i tn ->
        let loc = Map.find_exn ctx_buffers tn in
        let b = CArray.get arr i in
        setf b b_tn (Int32.of_int_exn tn.Tn.id);
        setf b b_pool (Int32.of_int_exn loc.pool_id);
        setf b b_off (Unsigned.UInt64.of_int loc.offset));
    let r = allocate vp null in
    check (c_link prior_context.device.dev.handle code.handle (CArray.start arr) n r);
    let routine = !@r in
    check (c_use_graph routine 1);
    let lowered_bindings : Indexing.lowered_bindings = List.map code.statics ~f:(fun s -> (s, ref 0)) in
    let work () =
      (* a negative or out-of-range value is reported as Utils.User_error by the library, as
         arrayjit/lib/cuda_backend.ml:1015-1030 does *)
      let vals = CArray.of_list int64_t (List.map lowered_bindings ~f:(fun (_, r) -> Int64.of_int !r)) in
      check (c_launch routine (CArray.start vals) (List.length lowered_bindings))
    in
    ( lowered_bindings,
      Task.Task { context_lifetime = (prior_context, routine); description = "launches " ^ code.name; work } )

  let link_batch prior_context code_batch ctx_buffers =
    let bindings = ref [] in
    let tasks =
      Array.mapi code_batch ~f:(fun i c ->
          Option.bind c ~f:(fun c ->
              Option.map ctx_buffers.(i) ~f:(fun bufs ->
                  let b, t = link prior_context c bufs in
                  bindings := b;
                  t)))
    in
    (!bindings, tasks)
end
