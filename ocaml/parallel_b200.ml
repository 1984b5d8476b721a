(* parallel_b200.ml — data-parallel training over the b200 backend with an NCCL gradient exchange.

   STATUS: source only, never compiled (no OCaml toolchain where this backend was built).  It states,
   in the reference's own terms, what replaces the exchange of [Parallel.data_parallel]
   (lib/parallel.ml:166-383) when the backend is "b200"; the same call sequence is exercised
   through the Python mirror (ocannl_b200/parallel.py: [data_parallel] / [Handle]) and its tests.

   What stays: the [Parallel.handle] record (lib/parallel.ml:112-141) with all its fields, the
   sharding of inputs and targets with [Parallel.shard_along] (:51-79), one loss graph per shard
   with seeds [base_seed + i] (:184-191), all shards held by this one process.

   What changes: the reference sums every parameter gradient on an "owner" shard through
   merge-buffer copies, runs the optimizer there and copies the parameters back to the others
   (:247-304: n_params x (n_shards - 1) transfers each way, serialised on the host).  Here
     - [grad_sync] is one grouped NCCL allreduce per parameter gradient over the shards' buffers
       ([b200_allreduce_all], sum or average), nothing passes through a merge buffer;
     - every shard runs its own optimizer routine on the reduced gradients, so the replicas stay
       equal without a broadcast (they start equal: the owner's initial parameters are copied to the
       other shards once, with plain device-to-device copies).
   With [Sum] and a sum-over-batch loss, or [Mean] and a mean loss, the result equals the one-shard
   run (test/training/data_parallel.ml:9-17). *)

open Base
open Ocannl
module Tn = Ir.Tnode
module B = B200_backend
open Ctypes

type reduction = Parallel.reduction = Sum | Mean

(* {pool, offset} of a node in a linked context (Backend_intf.context.ctx_buffers). *)
let loc_of (ctx : _ Ir.Backend_intf.context) (tn : Tn.t) = Map.find_exn ctx.ctx_buffers tn

let data_parallel ?(reduction = Mean) ?(weight_decay = 0.0) ?(momentum = 0.0) ?(base_seed = 0) ~n_shards
    ~(bindings : Ir.Indexing.unit_bindings) ~(learning_rate : Tensor.t) ~(inputs : Tensor.t) ~(targets : Tensor.t)
    ~(loss_of : Tensor.t -> Tensor.t -> Tensor.t) ~f () =
  if n_shards <= 0 then invalid_arg "Parallel.data_parallel: n_shards must be > 0";
  let backend = Backends.fresh_backend ~backend_name:"b200" () in
  let module Backend = (val backend : Ir.Backend_intf.Backend) in
  if Backend.num_devices () < n_shards then
    invalid_arg "Parallel_b200.data_parallel: one GPU per shard is needed (NCCL ranks must be distinct devices)";
  let xs = Parallel.shard_along ~axis:0 ~n_shards inputs and ys = Parallel.shard_along ~axis:0 ~n_shards targets in
  let shard_seeds = Array.init n_shards ~f:(fun i -> base_seed + i) in
  let losses =
    Tensor.with_saved_random_seed (fun () ->
        Array.mapi shard_seeds ~f:(fun i seed ->
            Tensor.set_random_seed ~seed ();
            loss_of xs.(i) ys.(i)))
  in
  let params = Array.map losses ~f:(fun l -> Array.of_list (Set.to_list l.Tensor.params)) in
  let n_params = Array.length params.(0) in
  (* per shard: context on its own device, parameters initialised, forward+backward linked, and --
     unlike the reference -- its OWN optimizer routine *)
  let devices = Array.init n_shards ~f:(fun i -> Backend.get_device ~ordinal:i) in
  let streams = Array.map devices ~f:Backend.new_stream in
  let link_on ctx comp = Backend.link ctx (Backend.compile ctx.Ir.Backend_intf.optimize_ctx bindings comp) in
  let shards =
    Array.init n_shards ~f:(fun i ->
        let ctx = Backend.make_context ~optimize_ctx:(Backend.empty_optimize_ctx ()) streams.(i) in
        let init = link_on ctx (Tensor.init_params losses.(i)) in
        Train.run init;
        let update = link_on init.context (Train.grad_update ~setup_for_parallel:true losses.(i)) in
        let lr = link_on update.context (Tensor.init_params learning_rate) in
        Train.run lr;
        let sgd =
          link_on lr.context
            (Train.sgd_update ~learning_rate ~weight_decay
               ?momentum:(if Float.(momentum > 0.0) then Some momentum else None)
               losses.(i))
        in
        (update, sgd))
  in
  let ctx_of i = (snd shards.(i)).Ir.Backend_intf.context in
  (* replicas start from the owner's parameters: one device-to-device copy per parameter and shard *)
  for i = 1 to n_shards - 1 do
    Array.iteri params.(0) ~f:(fun k owner_p ->
        ignore
          (Backend.device_to_device owner_p.Tensor.value ~into_merge_buffer:No ~dst:(ctx_of i) ~src:(ctx_of 0)
             ~dst_loc:(Some (loc_of (ctx_of i) params.(i).(k).Tensor.value))))
  done;
  Array.iter streams ~f:Backend.await;
  (* the communicators of all shards at once (one process drives every device) *)
  let devs = CArray.of_list B.vp (Array.to_list (Array.map devices ~f:(fun d -> d.Ir.Backend_intf.dev.B.handle))) in
  let comms = CArray.make B.vp n_shards in
  if n_shards > 1 then B.check (B.c_comm_init_all n_shards (CArray.start devs) (CArray.start comms));
  let grad_of (p : Tensor.t) = (Option.value_exn p.Tensor.diff).Tensor.grad in
  let grad_sync () =
    if n_shards > 1 then
      for k = 0 to n_params - 1 do
        let pools = CArray.make int n_shards and offs = CArray.make size_t n_shards in
        for i = 0 to n_shards - 1 do
          let l = loc_of (ctx_of i) (grad_of params.(i).(k)) in
          CArray.set pools i l.Ir.Backend_intf.pool_id;
          CArray.set offs i (Unsigned.Size_t.of_int l.offset)
        done;
        let count = Tn.num_elems (grad_of params.(0).(k)) in
        (* gradients are single precision (dtype 0); op 0 = sum, 1 = average *)
        B.check
          (B.c_allreduce_all n_shards (CArray.start comms) (CArray.start pools) (CArray.start offs)
             (Unsigned.Size_t.of_int count) 0
             (match reduction with Sum -> 0 | Mean -> 1))
      done
  in
  let step () =
    Array.iter shards ~f:(fun (update, _) -> Train.run update);   (* every shard is queued before any wait *)
    grad_sync ();
    Array.iter shards ~f:(fun (_, sgd) -> Train.run sgd);
    Array.iter streams ~f:Backend.await
  in
  let read ctx stream tn =
    let nd = Ir.Ndarray.create_array ~debug:"parallel_b200" (Lazy.force tn.Tn.prec) ~dims:(Lazy.force tn.Tn.dims)
               ~padding:(Lazy.force tn.Tn.padding) in
    ignore (Backend.to_host ctx tn nd : bool);
    Backend.await stream;
    Ir.Ndarray.retrieve_flat_values nd
  in
  let set_batch ~inputs ~targets =
    let nxs = Parallel.shard_along ~axis:0 ~n_shards inputs and nys = Parallel.shard_along ~axis:0 ~n_shards targets in
    for i = 0 to n_shards - 1 do
      let up dst (src : Tensor.t) =
        ignore (Backend.from_host (ctx_of i) dst (Lazy.force (Option.value_exn (Ir.Host_inits.find src.Tensor.value))) : bool)
      in
      up xs.(i).Tensor.value nxs.(i);
      up ys.(i).Tensor.value nys.(i);
      Backend.await streams.(i)
    done
  in
  f
    {
      Parallel.n_shards;
      step;
      grad_sync;
      set_batch;
      owner_loss_value = (fun () -> (read (ctx_of 0) streams.(0) losses.(0).Tensor.value).(0));
      sync_params_to_host = (fun () -> Array.iter streams ~f:Backend.await);
      read_values = (fun t -> read (ctx_of 0) streams.(0) t.Tensor.value);
      owner_params = params.(0);
      shard_seeds;
    }
